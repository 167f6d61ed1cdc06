// Forward of dense varlen GQA attention with the strided-causal mask on the 5th-generation tensor
// cores (tcgen05.mma, accumulators in tensor memory).
//
// CTA = two row tiles A and B of 128 rows each; a row tile is (128/G consecutive query tokens) x (G query heads of one
// KV head); B holds the tokens right after A's.  Key tiles of 128 go through SMEM rings shared by both row tiles.
//   warp 8      : TMA producer (Q of tile A and the first K tile first, so that the first product starts early, then Q of
//                 tile B, K tiles through a ring of 3 and V tiles through a ring of 2)
//   warp 9      : allocates TMEM; issues, per key tile and row tile, S = Q K^T (SMEM x SMEM -> TMEM) and O += P V
//                 (P read from TMEM, V from SMEM MN-major), alternating between the two row tiles: while the softmax
//                 threads of one tile work, the tensor pipe runs the other tile's products
//   warps 0..3  : softmax of tile A, one thread per row (TMEM lane): a first pass over the 128 logits of the key tile
//                 finds the row maximum, a second pass reads them again, exponentiates and writes P as 16-bit pairs
//                 back into tensor memory over the logits, where the P V instruction reads its A operand -- P never
//                 touches shared memory.  (Full tiles of rows that already have a reference maximum take a single pass,
//                 see the loop.)  A lazily updated reference maximum is kept: O and l are rescaled only when the
//                 row maximum grows by more than 2^8.  At the end the threads normalise O and store it (through the tile's Q
//                 buffer and a TMA store when all of the tile's tokens belong to the sequence)
//   warps 4..7  : the same for tile B
// The tensor pipe executes one thread's MMAs in issue order, so S(i+1) of a row tile, issued after its P V(i), cannot
// overwrite P(i) before it has been read.
// TMEM columns: [0,128) S/P of A, [128,256) S/P of B, [256,256+D) O of A, [384,384+D) O of B.
#include <type_traits>

#include "attn_tile.cuh"
#include "dispatch.h"
#include "host_util.h"
#include "nsa_b200.h"
#include "tc5.cuh"

namespace nsa {

#ifndef NSA_POLY_EVERY
#define NSA_POLY_EVERY 3
#endif
constexpr int kPolyEvery = NSA_POLY_EVERY;  // one pair of exponentials in kPolyEvery is evaluated as a polynomial

struct DenseFwdTcParams {
  void* o;
  float* lse;  // [Nq, Hq]
  const int* cu_q;
  const int* cu_k;
  long long o_sn, o_sh;
  int B, Hq, Hkv, G, logG;
  int window, stride, causal;
  int left;  // >= 0: sliding window, a query also needs key >= t - left (plain causal mask only); < 0: no lower bound
  float scale2;
  Status st;
};

__device__ __forceinline__ int visible_keys_tc(int t, int Lk, int window, int stride, int causal) {
  if (!causal) return Lk;
  if (t < window - 1) return 0;
  return min(Lk, (t - window + 1) / stride + 1);
}

constexpr int kTcKeyTile = 128;
constexpr int kTcKStages = 3;  // a K tile is free as soon as both row tiles' Q K^T are done
constexpr int kTcVStages = 2;  // a V tile is free when both row tiles' P V are done

template <typename T, int D>
__global__ void __launch_bounds__(320, 1)
dense_fwd_tc_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                    const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmO, DenseFwdTcParams p) {
  constexpr int PANELS = D / 64;
  constexpr int PANEL_BYTES = 128 * 128;            // 128 rows x 128 B
  constexpr int Q_BYTES = 128 * D * 2;              // one row tile
  constexpr int KV_BYTES = kTcKeyTile * D * 2;      // one K or V tile
  extern __shared__ __align__(1024) uint8_t smem[];
  uint8_t* q_sm = smem;                             // [2] row tiles
  uint8_t* k_sm = q_sm + 2 * Q_BYTES;
  uint8_t* v_sm = k_sm + kTcKStages * KV_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(v_sm + kTcVStages * KV_BYTES);
  uint64_t* q_full = bars;
  uint64_t* k_full = bars + 1;
  uint64_t* k_empty = k_full + kTcKStages;
  uint64_t* v_full = k_empty + kTcKStages;
  uint64_t* v_empty = v_full + kTcVStages;
  uint64_t* s_full = v_empty + kTcVStages;   // [2] per row tile
  uint64_t* p_full = s_full + 2;             // [2]
  uint64_t* pv_done = p_full + 2;            // [2]
  uint64_t* qb_full = pv_done + 2;           // Q of row tile B (q_full covers tile A alone: the first product needs only it)
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(qb_full + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (smem_u32(smem) & 1023u) {  // the swizzled operand tiles need a 1024-byte aligned base
    if (threadIdx.x == 0) p.st.raise(kErrSmemLayout);
    return;
  }
  const int b = blockIdx.y, h = blockIdx.z;
  const int qs = __ldg(p.cu_q + b), Lq = __ldg(p.cu_q + b + 1) - qs;
  const int ksq = __ldg(p.cu_k + b), Lk = __ldg(p.cu_k + b + 1) - ksq;
  const int QT = 128 >> p.logG;  // tokens per row tile
  const int qt = gridDim.x - 1 - blockIdx.x;
  const int q0 = qt * 2 * QT;
  if (q0 >= Lq) return;
  const int t_hi = min(q0 + 2 * QT, Lq) - 1;
  // with a sliding window the first key tiles are invisible to every row of the CTA: start at tile kt0
  const int kt0 = p.left >= 0 ? max(0, q0 - p.left) / kTcKeyTile : 0;
  const int ntiles = max(0, (visible_keys_tc(t_hi, Lk, p.window, p.stride, p.causal) + kTcKeyTile - 1) / kTcKeyTile - kt0);

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    mbar_init(qb_full, 1);
    for (int s = 0; s < kTcKStages; ++s) {
      mbar_init(k_full + s, 1);
      mbar_init(k_empty + s, 1);
    }
    for (int s = 0; s < kTcVStages; ++s) {
      mbar_init(v_full + s, 1);
      mbar_init(v_empty + s, 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(s_full + s, 1);
      mbar_init(p_full + s, 4);
      mbar_init(pv_done + s, 1);
    }
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
      // Q of tile A and the first K tile arrive first (the first product can start), then Q of tile B
      mbar_expect_tx(q_full, Q_BYTES);
#pragma unroll
      for (int pn = 0; pn < PANELS; ++pn) tma_load_3d(q_sm + pn * PANEL_BYTES, &tmQ, q_full, pn * 64, h * p.G, qs + q0);
      // K runs one tile ahead of V: tile i's V is requested after tile i+1's K
      for (int i = 0; i <= ntiles; ++i) {
        if (i < ntiles) {
          const int s = i % kTcKStages;
          if (i >= kTcKStages) mbar_wait(k_empty + s, ((i / kTcKStages) - 1) & 1, p.st);
          mbar_expect_tx(k_full + s, KV_BYTES);
#pragma unroll
          for (int pn = 0; pn < PANELS; ++pn)
            tma_load_3d(k_sm + s * KV_BYTES + pn * PANEL_BYTES, &tmK, k_full + s, pn * 64, h, ksq + (kt0 + i) * kTcKeyTile);
        }
        if (i == 0) {
          mbar_expect_tx(qb_full, Q_BYTES);
#pragma unroll
          for (int pn = 0; pn < PANELS; ++pn)
            tma_load_3d(q_sm + Q_BYTES + pn * PANEL_BYTES, &tmQ, qb_full, pn * 64, h * p.G, qs + q0 + QT);
        }
        if (i >= 1) {
          const int j = i - 1, s = j % kTcVStages;
          if (j >= kTcVStages) mbar_wait(v_empty + s, ((j / kTcVStages) - 1) & 1, p.st);
          mbar_expect_tx(v_full + s, KV_BYTES);
#pragma unroll
          for (int pn = 0; pn < PANELS; ++pn)
            tma_load_3d(v_sm + s * KV_BYTES + pn * PANEL_BYTES, &tmV, v_full + s, pn * 64, h, ksq + (kt0 + j) * kTcKeyTile);
        }
      }
    }
  } else if (warp == 9) {
    // ===================== MMA issuer =====================
    // The whole warp runs the control flow converged; one elected lane issues (see tc5.cuh on why).
    if (ntiles > 0) {
      const uint32_t idesc_qk = umma_idesc<T>(128, kTcKeyTile, false, false);
      const uint32_t idesc_pv = umma_idesc<T>(128, D, false, true);
      const uint32_t q_addr = smem_u32(q_sm);
      // S of row tile g for key tile i; the second row tile's product releases the K stage
      auto issue_qk = [&](int i, int g) {
        const uint32_t k_addr = smem_u32(k_sm + (i % kTcKStages) * KV_BYTES);
        if (elect_one()) {
          umma_block_ss<D / 16, PANEL_BYTES>(tmem + (uint32_t)(g * 128), q_addr + g * Q_BYTES, k_addr, idesc_qk);
          if (g == 1) umma_commit(k_empty + (i % kTcKStages));
          umma_commit(s_full + g);
        }
        __syncwarp();
      };
      auto issue_pv = [&](int i, int g) {
        const uint32_t v_addr = smem_u32(v_sm + (i % kTcVStages) * KV_BYTES);
        const uint32_t p_tmem = tmem + (uint32_t)(g * 128);  // P overwrote the first 64 columns of the tile's S
        if (elect_one()) {
#pragma unroll
          for (int kk = 0; kk < kTcKeyTile / 16; ++kk)
            umma_ts(tmem + 256 + g * 128, p_tmem + kk * 8, umma_desc_mnmajor(v_addr + kk * 2048, PANEL_BYTES), idesc_pv, i > 0 || kk > 0);
          if (g == 1) umma_commit(v_empty + (i % kTcVStages));
          umma_commit(pv_done + g);
        }
        __syncwarp();
      };
      mbar_wait(q_full, 0, p.st);
      mbar_wait(k_full, 0, p.st);
      tc_fence_after_sync();
      issue_qk(0, 0);
      mbar_wait(qb_full, 0, p.st);
      tc_fence_after_sync();
      issue_qk(0, 1);
      for (int i = 0; i < ntiles; ++i) {
#pragma unroll
        for (int g = 0; g < 2; ++g) {
          mbar_wait(p_full + g, i & 1, p.st);
          if (g == 0) mbar_wait(v_full + (i % kTcVStages), (i / kTcVStages) & 1, p.st);
          tc_fence_after_sync();
          issue_pv(i, g);
          if (i + 1 < ntiles) {
            if (g == 0) {
              mbar_wait(k_full + ((i + 1) % kTcKStages), ((i + 1) / kTcKStages) & 1, p.st);
              tc_fence_after_sync();
            }
            issue_qk(i + 1, g);
          }
        }
      }
    }
  } else {
    // ===================== softmax: one thread per row; warps 0..3 row tile A, warps 4..7 row tile B =====================
    const int g = warp >> 2;
    const int row = (warp & 3) * 32 + lane;
    const int tpos = q0 + g * QT + (row >> p.logG);
    const int head = h * p.G + (row & (p.G - 1));
    const bool valid = tpos < Lq;
    const int nvis = valid ? visible_keys_tc(tpos, Lk, p.window, p.stride, p.causal) : 0;
    const uint32_t s_base = tmem + ((uint32_t)((warp & 3) * 32) << 16) + (uint32_t)(g * 128);
    const uint32_t o_base = tmem + ((uint32_t)((warp & 3) * 32) << 16) + 256u + (uint32_t)(g * 128);
    float m_ref = -INFINITY, l = 0.f;
    for (int i = 0; i < ntiles; ++i) {
      mbar_wait(s_full + g, i & 1, p.st);
      tc_fence_after_sync();
      const int lim = nvis - (kt0 + i) * kTcKeyTile;  // columns below lim are visible ...
      const int lo = p.left >= 0 ? tpos - p.left - (kt0 + i) * kTcKeyTile : 0;  // ... from column lo on
      // Key tiles that every row of the warp sees in full (all but those on the mask's edge) take a path without the
      // per-element mask instructions.
      const bool full = __all_sync(0xffffffffu, lim >= kTcKeyTile && lo <= 0);
      // The two-pass form: row maximum first, then the exponentials relative to the (possibly raised) reference.
      auto two_pass = [&]() {
        // ---- pass 1: row maximum of the raw logits (the scale is positive) ----
        float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
        auto pass1 = [&](auto masked_tag) {
          constexpr bool MASKED = decltype(masked_tag)::value;
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            uint32_t su[32];
            tmem_ld32(s_base + c * 32, su);
            tmem_ld_wait();
#pragma unroll
            for (int j = 0; j < 32; j += 2) {
              const float v0 = (!MASKED || (c * 32 + j < lim && c * 32 + j >= lo)) ? __uint_as_float(su[j]) : -INFINITY;
              const float v1 = (!MASKED || (c * 32 + j + 1 < lim && c * 32 + j + 1 >= lo)) ? __uint_as_float(su[j + 1]) : -INFINITY;
              mx4[(j >> 1) & 3] = fmax3(mx4[(j >> 1) & 3], v0, v1);
            }
          }
        };
        if (full) pass1(std::false_type{}); else pass1(std::true_type{});
        const float mt = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3])) * p.scale2;
        const bool need = mt > m_ref + 8.f;
        float factor = 1.f;
        if (need) {
          factor = (m_ref == -INFINITY) ? 0.f : fast_exp2(m_ref - mt);
          m_ref = mt;
          l *= factor;
        }
        if (i > 0 && __any_sync(0xffffffffu, need)) {
          mbar_wait(pv_done + g, (i - 1) & 1, p.st);  // P V of the previous key tile is complete: O is stable
          tc_fence_after_sync();
#pragma unroll
          for (int c = 0; c < D / 32; ++c) {
            uint32_t r[32];
            tmem_ld32(o_base + c * 32, r);
            tmem_ld_wait();
#pragma unroll
            for (int j = 0; j < 32; j += 2) {
              const float2 y = fmul2(make_float2(__uint_as_float(r[j]), __uint_as_float(r[j + 1])), make_float2(factor, factor));
              r[j] = __float_as_uint(y.x);
              r[j + 1] = __float_as_uint(y.y);
            }
            tmem_st32(o_base + c * 32, r);
          }
          tmem_st_wait();
        }
        // ---- pass 2: P = exp2(S*scale - m_ref) as 16-bit pairs over the logits: the 32 columns of chunk c become the 16
        // packed columns [16c, 16c+16), which lie inside chunk c/2 -- already consumed when chunk c is written ----
        const float nm = (m_ref == -INFINITY) ? 0.f : -m_ref;
        float2 ls2[2] = {make_float2(0.f, 0.f), make_float2(0.f, 0.f)};
        auto pass2 = [&](auto masked_tag) {
          constexpr bool MASKED = decltype(masked_tag)::value;
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            uint32_t su[32];
            tmem_ld32(s_base + c * 32, su);
            tmem_ld_wait();
            uint32_t pk[16];
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              const float2 x = ffma2(make_float2(__uint_as_float(su[2 * j]), __uint_as_float(su[2 * j + 1])), make_float2(p.scale2, p.scale2),
                                     make_float2(nm, nm));
              float p0, p1;
              if (MASKED) {
                p0 = masked_exp2(c * 32 + 2 * j < lim && c * 32 + 2 * j >= lo, x.x);
                p1 = masked_exp2(c * 32 + 2 * j + 1 < lim && c * 32 + 2 * j + 1 >= lo, x.y);
              } else if (j % kPolyEvery == kPolyEvery - 1) {  // a share of the exponentials runs on the FMA pipe
                const float2 e = exp2_poly2(x);
                p0 = e.x;
                p1 = e.y;
              } else {
                p0 = fast_exp2(x.x);
                p1 = fast_exp2(x.y);
              }
              ls2[j & 1] = fadd2(ls2[j & 1], make_float2(p0, p1));
              pk[j] = DT<T>::pack(p0, p1);
            }
            tmem_st16(s_base + c * 16, pk);
          }
        };
        if (full) pass2(std::false_type{}); else pass2(std::true_type{});
        tmem_st_wait();
        l += (ls2[0].x + ls2[0].y) + (ls2[1].x + ls2[1].y);
      };
      // Full tiles of rows that already have a reference maximum are tried in ONE pass over the logits: exponentials
      // relative to the current reference, with the maximum of the exponents tracked on the side.  If no row of the
      // warp outgrew its reference by more than 2^8 -- the same test the two-pass form makes -- the packed P is stored
      // and the pass for the maximum (four more TMEM loads) was saved; otherwise nothing has been written yet, the
      // logits are intact, and the tile is redone in two passes.  Both routes give the same P and the same sums.
      bool done = false;
      if (full && __all_sync(0xffffffffu, m_ref != -INFINITY)) {
        const float nm = -m_ref;
        uint32_t pk[64];
        float2 ls2[2] = {make_float2(0.f, 0.f), make_float2(0.f, 0.f)};
        float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          uint32_t su[32];
          tmem_ld32(s_base + c * 32, su);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            const float2 x = ffma2(make_float2(__uint_as_float(su[2 * j]), __uint_as_float(su[2 * j + 1])), make_float2(p.scale2, p.scale2),
                                   make_float2(nm, nm));
            mx4[j & 3] = fmax3(mx4[j & 3], x.x, x.y);
            float p0, p1;
            if (j % kPolyEvery == kPolyEvery - 1) {
              const float2 e = exp2_poly2(x);
              p0 = e.x;
              p1 = e.y;
            } else {
              p0 = fast_exp2(x.x);
              p1 = fast_exp2(x.y);
            }
            ls2[j & 1] = fadd2(ls2[j & 1], make_float2(p0, p1));
            pk[c * 16 + j] = DT<T>::pack(p0, p1);
          }
        }
        const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
        if (!__any_sync(0xffffffffu, mx > 8.f)) {
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            uint32_t pc[16];
#pragma unroll
            for (int j = 0; j < 16; ++j) pc[j] = pk[c * 16 + j];
            tmem_st16(s_base + c * 16, pc);
          }
          tmem_st_wait();
          l += (ls2[0].x + ls2[0].y) + (ls2[1].x + ls2[1].y);
          done = true;
        }
      }
      if (!done) two_pass();
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(p_full + g);
    }
    // ---- epilogue: O / l ----
    if (ntiles > 0) {
      mbar_wait(pv_done + g, (ntiles - 1) & 1, p.st);
      tc_fence_after_sync();
    }
    const float inv = l > 0.f ? 1.f / l : 0.f;
    if (valid) p.lse[(long long)(qs + tpos) * p.Hq + head] = l > 0.f ? m_ref + log2f(l) : -INFINITY;
    // A row tile whose tokens all belong to the sequence leaves through shared memory (its own Q buffer, free since its
    // last S product, in the swizzled panel layout) and one TMA store per panel; otherwise row by row.
    const bool staged = ntiles > 0 && q0 + g * QT + QT <= Lq;
    T* orow = static_cast<T*>(p.o) + (long long)(qs + tpos) * p.o_sn + (long long)head * p.o_sh;
#pragma unroll
    for (int c = 0; c < D / 32; ++c) {
      uint32_t r[32];
      if (ntiles > 0) {
        tmem_ld32(o_base + c * 32, r);
        tmem_ld_wait();
      } else {
#pragma unroll
        for (int j = 0; j < 32; ++j) r[j] = 0u;
      }
      if (staged) {
        const uint32_t stage = smem_u32(q_sm + g * Q_BYTES);
#pragma unroll
        for (int q4 = 0; q4 < 4; ++q4) {
          const int ci = c * 4 + q4;  // 16-byte chunk of the row
          const uint32_t off = (ci >> 3) * PANEL_BYTES + row * 128 + (((ci & 7) ^ (row & 7)) << 4);
          asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};\n" ::"r"(stage + off),
                       "r"(DT<T>::pack(__uint_as_float(r[q4 * 8 + 0]) * inv, __uint_as_float(r[q4 * 8 + 1]) * inv)),
                       "r"(DT<T>::pack(__uint_as_float(r[q4 * 8 + 2]) * inv, __uint_as_float(r[q4 * 8 + 3]) * inv)),
                       "r"(DT<T>::pack(__uint_as_float(r[q4 * 8 + 4]) * inv, __uint_as_float(r[q4 * 8 + 5]) * inv)),
                       "r"(DT<T>::pack(__uint_as_float(r[q4 * 8 + 6]) * inv, __uint_as_float(r[q4 * 8 + 7]) * inv)) : "memory");
        }
      } else if (valid) {
#pragma unroll
        for (int q4 = 0; q4 < 4; ++q4) {
          uint4 out;
          out.x = DT<T>::pack(__uint_as_float(r[q4 * 8 + 0]) * inv, __uint_as_float(r[q4 * 8 + 1]) * inv);
          out.y = DT<T>::pack(__uint_as_float(r[q4 * 8 + 2]) * inv, __uint_as_float(r[q4 * 8 + 3]) * inv);
          out.z = DT<T>::pack(__uint_as_float(r[q4 * 8 + 4]) * inv, __uint_as_float(r[q4 * 8 + 5]) * inv);
          out.w = DT<T>::pack(__uint_as_float(r[q4 * 8 + 6]) * inv, __uint_as_float(r[q4 * 8 + 7]) * inv);
          *reinterpret_cast<uint4*>(orow + c * 32 + q4 * 8) = out;
        }
      }
    }
    if (staged) {
      fence_proxy_async();  // the TMA engine reads the tile through the async proxy
      asm volatile("bar.sync %0, 128;\n" ::"r"(1 + g) : "memory");
      if ((warp & 3) == 0 && lane == 0) {
#pragma unroll
        for (int pn = 0; pn < PANELS; ++pn) tma_store_3d(&tmO, q_sm + g * Q_BYTES + pn * PANEL_BYTES, pn * 64, h * p.G, qs + q0 + g * QT);
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
static int launch_dense_fwd_tc(const void* q, const void* k, const void* v, const long long* S, int Nq, int Nk, int max_seqlen_q,
                               DenseFwdTcParams p, cudaStream_t stream) {
  // S: q_n q_h k_n k_h v_n v_h o_n o_h
  CUtensorMap tmQ, tmK, tmV;
  const int QT = 128 / p.G;
  int rc = make_tmap_3d(&tmQ, DT<T>::kTmapType, q, D, p.Hq, Nq, S[1], S[0], 64, p.G, QT);
  if (rc) return rc;
  rc = make_tmap_3d(&tmK, DT<T>::kTmapType, k, D, p.Hkv, Nk, S[3], S[2], 64, 1, kTcKeyTile);
  if (rc) return rc;
  rc = make_tmap_3d(&tmV, DT<T>::kTmapType, v, D, p.Hkv, Nk, S[5], S[4], 64, 1, kTcKeyTile);
  if (rc) return rc;
  CUtensorMap tmO;
  rc = make_tmap_3d(&tmO, DT<T>::kTmapType, p.o, D, p.Hq, Nq, p.o_sh, p.o_sn, 64, p.G, QT);
  if (rc) return rc;
  const size_t smem = 2 * 128 * D * 2 + (kTcKStages + kTcVStages) * kTcKeyTile * D * 2 + 32 * sizeof(uint64_t);
  auto kern = dense_fwd_tc_kernel<T, D>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return cuda_rc(e);
  dim3 grid((max_seqlen_q + 2 * QT - 1) / (2 * QT), p.B, p.Hkv);
  { LaunchScope ls_("dense_fwd_tc", stream); kern<<<grid, 320, smem, stream>>>(tmQ, tmK, tmV, tmO, p); }
  return cuda_rc(cudaGetLastError());
}

// entry used by nsa_varlen_attn_fwd (dense_fwd.cu)
int varlen_attn_fwd_tc(const void* q, const void* k, const void* v, const int* cu_q, const int* cu_k, void* o, float* lse,
                       int total_q, int total_k, int batch, int max_seqlen_q, int Hq, int Hkv, int head_dim, int causal,
                       int window, int stride, int left, const long long* strides, float sm_scale, int dtype, cudaStream_t stream) {
  DenseFwdTcParams p;
  p.o = o; p.lse = lse; p.cu_q = cu_q; p.cu_k = cu_k;
  p.o_sn = strides[6]; p.o_sh = strides[7];
  p.B = batch; p.Hq = Hq; p.Hkv = Hkv; p.G = Hq / Hkv;
  p.logG = 0;
  while ((1 << p.logG) < p.G) ++p.logG;
  p.window = window; p.stride = stride; p.causal = causal; p.left = left;
  p.scale2 = sm_scale * kLog2e;
  p.st.word = status_word();
  return NSA_DISPATCH_T_D(dtype, head_dim, launch_dense_fwd_tc, q, k, v, strides, total_q, total_k, max_seqlen_q, p, stream);
}

}  // namespace nsa
