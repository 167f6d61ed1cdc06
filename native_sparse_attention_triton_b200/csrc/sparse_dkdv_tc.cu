// dK/dV pass of the top-k sparse attention on the 5th-generation tensor cores (head_dim 128).
//
// Work item = one tile of 64 keys of a selected block (K and V tile resident in SMEM) x a stream of row tiles taken from
// the block's inverted index (the tokens that selected it); a row tile is 128 rows = (128/G tokens) x (G query
// heads).  All four products have M = 128:
//     S    = Q  K^T          [128 rows x 64 keys]   A = Q  (K-major),  B = K tile (K-major)
//     dP   = dO V^T          [128 rows x 64 keys]   A = dO (K-major),  B = V tile (K-major)
//     dV^T = dO^T P          [128 d    x 64 keys]   A = dO (MN-major), B = P  [rows][keys] (MN-major)
//     dK^T = Q^T  dS         [128 d    x 64 keys]   A = Q  (MN-major), B = dS [rows][keys] (MN-major)
//     dQ^T = K^T  dS^T       [128 d    x 128 rows]  A = K tile (MN-major), B = dS [rows][keys] (K-major)   (optional)
// so the token/head rows are the reduction dimension of dV and dK and the G heads of a KV group are summed
// inside the MMA.  S and dP are double-buffered in TMEM; dV^T and dK^T stay in TMEM for the whole CTA and are added
// to the fp32 accumulators in global memory at the end.
//
// With p.dq32 set the pass also produces dQ: the K tile is already resident and dS already sits in shared memory, so
// the contribution of this key tile to the rows' dQ costs one more product (4 MMAs of 128 x 128 x 16) and no operand
// traffic.  A per-token kernel would fetch the 64-key tile again for every token that selected it (32 KB per token and
// block through the L2-to-SM path, the bound of such a kernel); here the tile is shared by every token of the list and
// what leaves the SM is the 128 x 128 fp32 partial result, added to the dQ accumulator with red.global.add.f32.  The
// product is computed TRANSPOSED (d on the TMEM lanes) so that the 32 lanes of a warp hold 32 consecutive d of one
// (token, head) row: one reduction instruction then covers one whole 128-byte line.  Measured on this part, reductions
// into L2-resident lines run at 5.2 TB/s when a warp instruction covers whole lines (scalar or v4 alike), 2.8 TB/s when
// each lane hits its own line (a thread owning a row), and 2.5 TB/s when the lines live in HBM: the work items are
// ordered by token window (index_scan) so that the accumulator rows being reduced into stay resident in L2.
//
// The rows of a tile are scattered tokens (4 KB of Q and of dO each).  One TMA box per token tops out near
// 26 bytes/clock/SM (the box rate), so the rows are gathered with 16-byte cp.async instead (more than 60
// bytes/clock/SM) by four loader warps, two per tile parity, into the same 128-byte-swizzled layout TMA would write.
// The Q ring has three stages (a Q tile lives from its S product to its dK product), the dO ring two: dP(i) is
// issued right behind S(i) and dV(i) as soon as P(i) is there, which needs only S(i), so dO(i) is released early.
//   warps 0..7  : two threads per row (32 of the 64 key columns each).  P phase (after S): P = exp2(S*scale - lse)
//                 -> 16-bit SMEM tile; dS phase (after dP): dS = P (dP - delta) scale -> SMEM tile.  The per-row
//                 (lse, delta) come straight from global memory, fetched one tile ahead.  At the end they drain
//                 dV / dK from TMEM
//   warps 8..11 : cp.async loaders (warps 8,9: even tiles; 10,11: odd tiles)
//   warp 12     : TMEM allocation, K/V TMA, MMA issue (converged warp, one elected lane issues)
//   warps 13..16: dQ drain (only with p.dq32): warp w owns the TMEM lanes (= d) of quarter w % 4 and adds the 128 rows of
//                 every tile's dQ^T to the fp32 accumulator.  They are warps of their own because the reductions are the
//                 slower of the two streams of this kernel (64 KB per tile at about 19 bytes/clock/SM of L2 reduction
//                 throughput against 2900 clocks of products): issued from the softmax warps they stalled the P and dS
//                 phases behind every full reduction queue and the two costs added up (11.6 ms at 64 K tokens; 10.1 ms
//                 with these warps, of which 8.5 ms remain when the reductions are left out).
// TMEM columns: S0 [0,64) S1 [64,128) dP0 [128,192) dP1 [192,256) dV^T [256,320) dK^T [320,384) dQ [384,512).
#include <algorithm>

#include "attn_bwd.h"
#include "host_util.h"
#include "tc5.cuh"

namespace nsa {

namespace {
constexpr int kSpQStages = 3;
constexpr int kSpDoStages = 2;
constexpr int kSpRowBytes = 128 * 128 * 2;  // Q or dO rows of one tile: 32 KB, 2 panels of [128 rows][64 d]
constexpr int kSpRowPanel = 128 * 128;
constexpr int kSpKvBytes = 64 * 128 * 2;    // K or V tile: 16 KB, 2 panels of [64 keys][64 d]
constexpr int kSpKvPanel = 64 * 128;
constexpr int kSpPdBytes = 128 * 64 * 2;    // P or dS tile [128 rows][64 keys]: one panel
constexpr int kSpThreads = 17 * 32;
constexpr int kSpItemQ = 4;                // entries of a CTA's queue of work items

__device__ __forceinline__ void red_add1(float* dst, uint32_t v) {
  asm volatile("red.global.add.f32 [%0], %1;\n" ::"l"(dst), "f"(__uint_as_float(v)) : "memory");
}
}  // namespace

// One work item: a 64-key tile of a selected block and (a chunk of) the list of tokens that selected the block.
struct SpItem {
  int h, qs, kpos, krow0, kvalid, tok_begin, tok_count;
  int ntiles;  // 0: nothing to do (past the end of the sequence, or an empty chunk)
};

// loads whose place in the instruction stream is kept: an item's description is fetched while the item before it is
// being processed
__device__ __forceinline__ int ld_i32_here(const int* ptr) {
  int v;
  asm volatile("ld.global.nc.b32 %0, [%1];\n" : "=r"(v) : "l"(ptr));
  return v;
}

template <typename T, int LOGG>
__global__ void __launch_bounds__(kSpThreads, 1)
sparse_dkdv_tc_kernel(const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV, const T* __restrict__ q,
                      const T* __restrict__ dout, long long q_sn, long long q_sh, long long do_sn, long long do_sh, DkdvParams p) {
  constexpr int logG = LOGG;
  constexpr int G = 1 << LOGG;
  constexpr int D = 128;
  constexpr int KT = 64;
  extern __shared__ __align__(1024) uint8_t smem[];
  uint8_t* k_sm = smem;
  uint8_t* v_sm = k_sm + kSpKvBytes;
  uint8_t* p_sm = v_sm + kSpKvBytes;
  uint8_t* ds_sm = p_sm + kSpPdBytes;
  uint8_t* q_ring = ds_sm + kSpPdBytes;
  uint8_t* do_ring = q_ring + kSpQStages * kSpRowBytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(do_ring + kSpDoStages * kSpRowBytes);
  uint64_t* kv_full = bars;
  uint64_t* q_full = bars + 1;
  uint64_t* q_empty = q_full + kSpQStages;
  uint64_t* do_full = q_empty + kSpQStages;
  uint64_t* do_empty = do_full + kSpDoStages;
  uint64_t* s_full = do_empty + kSpDoStages;  // [2]
  uint64_t* s_empty = s_full + 2;             // [2]
  uint64_t* dp_full = s_empty + 2;            // [2]
  uint64_t* dp_empty = dp_full + 2;           // [2]
  uint64_t* p_full = dp_empty + 2;
  uint64_t* p_empty = p_full + 1;
  uint64_t* ds_full = p_empty + 1;
  uint64_t* ds_empty = ds_full + 1;
  uint64_t* all_done = ds_empty + 1;
  uint64_t* dq_full = all_done + 1;
  uint64_t* dq_empty = dq_full + 1;
  uint64_t* acc_free = dq_empty + 1;          // the dV / dK accumulators of the previous item have been read out
  uint64_t* iq_full = acc_free + 1;           // [kSpItemQ] an entry of the CTA's item queue has been published
  uint64_t* iq_empty = iq_full + kSpItemQ;    // [kSpItemQ] all 17 warps have read it
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(iq_empty + kSpItemQ);
  volatile int* item_q = reinterpret_cast<volatile int*>(tmem_slot + 2);   // [kSpItemQ] item ids handed out by the grid-wide counter
  const bool with_dq = p.dq32 != nullptr;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int TPT = 128 >> logG;  // tokens per row tile
  if (smem_u32(smem) & 1023u) {  // the swizzled operand tiles need a 1024-byte aligned base
    if (threadIdx.x == 0) p.st.raise(kErrSmemLayout);
    return;
  }

  // ---- the CTA is persistent: it takes items from a grid-wide counter, in list order ----
  // (In order, because the list is sorted by token window: CTAs that run together then reduce into the same L2-resident part
  // of the dQ accumulator.  A fixed stride per CTA let them drift windows apart: 15.8 ms against 10.2 ms.)  One lane fetches
  // the CTA's next item id and publishes it in a small shared-memory queue that all 17 warps read, each at its own pace.
  // Tensor memory, barriers and the warps' roles are set up once; the rings, the TMEM buffers and every barrier phase run
  // on across items (tile index j counts the tiles of all items of this CTA), so that the gathers, the first logits and the
  // P phase of an item overlap the last products and the dV / dK read-out of the item before it.
  const int total_x = p.Hkv * p.NW * p.TB;
  const int nsub = p.block_size / KT;                          // 64-key tiles per selected block
  const int n_items = __ldg(p.item_base + total_x) * nsub;     // work items: (entry of the list, tile of the block)
  if (n_items <= 0) return;
  auto load_item = [&](int work) -> SpItem {
    SpItem it;
    const int item = work / nsub, ysub = work - item * nsub;
    const int x = ld_i32_here(p.item_bin + item);  // the item's bin, written by index_scan
    const int base = ld_i32_here(p.item_base + x), off0 = ld_i32_here(p.offsets + x), off1 = ld_i32_here(p.offsets + x + 1);
    it.h = x / (p.NW * p.TB);
    const int gb = x % p.TB;
    const int b = find_sequence(p.cu_blocks, p.B, gb);
    it.qs = ld_i32_here(p.cu_q + b);
    const int Lq = ld_i32_here(p.cu_q + b + 1) - it.qs;
    const int blk = gb - ld_i32_here(p.cu_blocks + b);
    it.kpos = blk * p.block_size + ysub * KT;
    it.krow0 = it.qs + it.kpos;
    it.kvalid = min(KT, Lq - it.kpos);
    const int c = item - base;
    it.tok_begin = off0 + c * p.chunk;
    it.tok_count = min(p.chunk, (off1 - off0) - c * p.chunk);
    it.ntiles = (it.kvalid > 0 && it.tok_count > 0) ? (it.tok_count + TPT - 1) / TPT : 0;
    return it;
  };

  if (threadIdx.x == 0) {
    mbar_init(kv_full, 1);
    for (int s = 0; s < kSpQStages; ++s) {
      mbar_init(q_full + s, 64);
      mbar_init(q_empty + s, 1);
    }
    for (int s = 0; s < kSpDoStages; ++s) {
      mbar_init(do_full + s, 64);
      mbar_init(do_empty + s, 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(s_full + s, 1);
      mbar_init(s_empty + s, 8);
      mbar_init(dp_full + s, 1);
      mbar_init(dp_empty + s, 8);
    }
    mbar_init(p_full, 8);
    mbar_init(p_empty, 1);
    mbar_init(ds_full, 8);
    mbar_init(ds_empty, with_dq ? 2 : 1);  // dK, and dQ when it is produced, read the dS tile
    mbar_init(all_done, 1);
    mbar_init(dq_full, 1);
    mbar_init(dq_empty, 4);
    mbar_init(acc_free, 8);
    for (int s = 0; s < kSpItemQ; ++s) {
      mbar_init(iq_full + s, 1);
      mbar_init(iq_empty + s, kSpThreads / 32);
    }
    fence_barrier_init();
  }
  if (warp == 12) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = *reinterpret_cast<volatile uint32_t*>(tmem_slot);

  // k-th item of this CTA: published by lane 0 of warp 8 (publish), read once by every warp (take).  An id >= n_items
  // ends the sequence.
  auto publish = [&](int k) {
    const int s = k % kSpItemQ;
    if (k >= kSpItemQ) mbar_wait(iq_empty + s, ((k / kSpItemQ) - 1) & 1, p.st);
    item_q[s] = atomicAdd(p.item_counter, 1);
    mbar_arrive(iq_full + s);
  };
  auto take = [&](int k) -> int {
    const int s = k % kSpItemQ;
    mbar_wait(iq_full + s, (k / kSpItemQ) & 1, p.st);
    const int v = item_q[s];
    __syncwarp();
    if (lane == 0) mbar_arrive(iq_empty + s);
    return v;
  };
  auto item_or_none = [&](int item) -> SpItem {
    SpItem it;
    it.ntiles = 0;
    if (item < n_items) it = load_item(item);
    return it;
  };

  // every role walks the same list of items; `gt` is the number of tiles of the items before the current one
  if (warp >= 8 && warp < 12) {
    // ===================== loaders: group 0 (warps 8,9) tiles with even j, group 1 (warps 10,11) odd j =====================
    const int grp = (warp - 8) >> 1;
    const int tl = threadIdx.x - (8 + 2 * grp) * 32;  // 0..63
    const int chunk16 = tl & 15;                      // which 16 bytes of the row's 256
    const int row_in_step = tl >> 4;                  // 4 rows per step
    const uint32_t pn_off = (chunk16 >> 3) * kSpRowPanel;
    const int c8 = chunk16 & 7;
    int gt = 0;
    const bool publisher = warp == 8 && lane == 0;
    bool published_end = false;
    if (publisher) publish(0);
    int item = take(0);
    SpItem cur = item_or_none(item);
    for (int k = 0; item < n_items; ++k) {
      if (publisher && !published_end) {
        publish(k + 1);
        published_end = item_q[(k + 1) % kSpItemQ] >= n_items;
      }
      __syncwarp();
      const int nitem = take(k + 1);
      const SpItem nxt = item_or_none(nitem);
      if (cur.ntiles > 0) {
        const int ntiles = cur.ntiles, tok_begin = cur.tok_begin, tok_count = cur.tok_count, h = cur.h;
        // token ids of a tile: lane t of every loader warp holds the id of the tile's t-th token (at most 32 tokens per
        // tile), fetched one round ahead so that the gather itself has no dependent global load in front of it
        auto tile_tokens = [&](int i) {
          const int ti = i * TPT + lane;
          return (i < ntiles && lane < TPT && ti < tok_count) ? __ldg(p.list + tok_begin + ti) : -1;
        };
        const long long q_row0 = (long long)(h * p.G) * q_sh + chunk16 * 8, do_row0 = (long long)(h * p.G) * do_sh + chunk16 * 8;
        const int i0 = ((gt & 1) == grp) ? 0 : 1;
        int my_n = tile_tokens(i0);
        for (int i = i0; i < ntiles; i += 2) {
          const int j = gt + i;
          const int next_n = tile_tokens(i + 2);
          // Row r = slot * G + 4 * jj + row_in_step of the tile comes from token `slot`, head r % G.  Everything that does
          // not depend on the token is folded into constants so that a copy costs a handful of instructions.
          auto gather = [&](const T* src, long long sn, long long sh, long long row0, uint32_t dst_base) {
            const uint32_t dst0 = dst_base + pn_off + row_in_step * 128;
            const uint32_t sw0 = (uint32_t)((c8 ^ row_in_step) << 4), sw1 = (uint32_t)((c8 ^ (row_in_step + 4)) << 4);
            const T* src0 = src + row0 + (long long)row_in_step * sh;
#pragma unroll 4
            for (int slot = 0; slot < (128 >> LOGG); ++slot) {
              const int n = __shfl_sync(0xffffffffu, my_n, slot);
              const bool ok = n >= 0;
              const T* g = src0 + (long long)(ok ? n : 0) * sn;
#pragma unroll
              for (int jj = 0; jj < G / 4; ++jj) {
                const int jr = slot * (G / 4) + jj;  // r = 4 jr + row_in_step; r & 7 = row_in_step + 4 (jr & 1)
                cp_async16(dst0 + jr * 512 + ((jr & 1) ? sw1 : sw0), g + (long long)(4 * jj) * sh, ok);  // missing tokens: zero fill
              }
            }
          };
          const int sq = j % kSpQStages, sd = j % kSpDoStages;
          if (j >= kSpQStages) mbar_wait(q_empty + sq, ((j / kSpQStages) - 1) & 1, p.st);
          gather(q, q_sn, q_sh, q_row0, smem_u32(q_ring + sq * kSpRowBytes));
          cp_async_commit();
          if (j >= kSpDoStages) mbar_wait(do_empty + sd, ((j / kSpDoStages) - 1) & 1, p.st);
          gather(dout, do_sn, do_sh, do_row0, smem_u32(do_ring + sd * kSpRowBytes));
          cp_async_commit();
          cp_async_wait<1>();
          fence_proxy_async();  // the tensor pipe reads these bytes through the async proxy
          mbar_arrive(q_full + sq);
          cp_async_wait<0>();
          fence_proxy_async();
          mbar_arrive(do_full + sd);
          my_n = next_n;
        }
        gt += ntiles;
      }
      cur = nxt;
      item = nitem;
    }
  } else if (warp == 12) {
    // ===================== K/V load and MMA issue (converged warp, elected lane issues) =====================
    const uint32_t idesc_s = umma_idesc<T>(128, KT, false, false);
    const uint32_t idesc_t = umma_idesc<T>(128, KT, true, true);
    const uint32_t k_addr = smem_u32(k_sm), v_addr = smem_u32(v_sm), p_addr = smem_u32(p_sm), ds_addr = smem_u32(ds_sm);
    const uint32_t q_base = smem_u32(q_ring), do_base = smem_u32(do_ring);
    // S/dP: A = rows (two [128][64] panels), B = K or V tile (two [64][64] panels)
    auto issue_logits = [&](uint32_t a_addr, uint32_t b_addr, uint32_t d_tmem, uint64_t* bar) {
      if (elect_one()) {
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk)
          umma_ss(d_tmem, umma_desc_kmajor(a_addr + (kk >> 2) * kSpRowPanel + (kk & 3) * 32),
                  umma_desc_kmajor(b_addr + (kk >> 2) * kSpKvPanel + (kk & 3) * 32), idesc_s, kk > 0);
        umma_commit(bar);
      }
      __syncwarp();
    };
    // dV^T/dK^T: reduction over the 128 rows, 16 at a time; A = rows MN-major (d as M), B = P or dS tile MN-major
    auto issue_grad = [&](uint32_t a_addr, uint32_t b_addr, uint32_t d_tmem, bool first, uint64_t* bar_rows, uint64_t* bar_tile) {
      if (elect_one()) {
        umma_ss(d_tmem, umma_desc_mnmajor(a_addr, kSpRowPanel), umma_desc_mnmajor(b_addr, kSpPdBytes), idesc_t, !first);
#pragma unroll
        for (int kk = 1; kk < 128 / 16; ++kk)
          umma_ss(d_tmem, umma_desc_mnmajor(a_addr + kk * 2048, kSpRowPanel), umma_desc_mnmajor(b_addr + kk * 2048, kSpPdBytes),
                  idesc_t, true);
        umma_commit(bar_rows);
        umma_commit(bar_tile);
      }
      __syncwarp();
    };
    // dQ^T = K^T dS^T: A = K tile MN-major (d as M over two panels, 16 keys = 2048 bytes), B = dS tile K-major (one panel)
    const uint32_t idesc_q = umma_idesc<T>(128, 128, true, false);
    auto issue_dq = [&](uint32_t d_tmem) {
      if (elect_one()) {
#pragma unroll
        for (int kk = 0; kk < KT / 16; ++kk)
          umma_ss(d_tmem, umma_desc_mnmajor(k_addr + kk * 2048, kSpKvPanel), umma_desc_kmajor(ds_addr + kk * 32), idesc_q, kk > 0);
        umma_commit(dq_full);
        umma_commit(ds_empty);
      }
      __syncwarp();
    };
    // Five queues share the tensor pipe: S(j) and dP(j) need their rows and a free TMEM buffer; dV(j) needs P(j) (and
    // comes after dP(j), so that its completion can release the dO stage); dK(j) and dQ(j) need dS(j), dQ(j) also that
    // dQ(j-1) has been read out of its (single) TMEM buffer.  The counters run on across items.
    int ns = 0, np = 0, nv = 0, nk = 0, nq = 0;
    int gt = 0, n_done = 0;  // tiles of the items before this one; items processed
    bool alive = true;
    int item = take(0);
    SpItem cur = item_or_none(item);
    for (int k = 0; item < n_items && alive; ++k) {
      const int nitem = take(k + 1);
      const SpItem nxt = item_or_none(nitem);
      if (cur.ntiles > 0) {
        // every product of the item before has completed (waited for at its end): its K/V tile can be replaced
        if (elect_one()) {
          mbar_expect_tx(kv_full, 2 * kSpKvBytes);
#pragma unroll
          for (int pn = 0; pn < 2; ++pn) {
            tma_load_3d(k_sm + pn * kSpKvPanel, &tmK, kv_full, pn * 64, cur.h, cur.krow0);
            tma_load_3d(v_sm + pn * kSpKvPanel, &tmV, kv_full, pn * 64, cur.h, cur.krow0);
          }
        }
        __syncwarp();
        const int end = gt + cur.ntiles;
        if (!with_dq) nq = end;
        // dV^T / dK^T restart from zero with this item: not before the softmax warps have read out the previous item's
        bool acc_ok = n_done == 0;
        if (!mbar_wait(kv_full, n_done & 1, p.st)) alive = false;
        long long t0 = 0;
        int idle = 0;
        while (alive && (nk < end || nq < end)) {
          bool progressed = false;
          if (!acc_ok) acc_ok = mbar_test(acc_free, (n_done - 1) & 1);
          if (nq < np && nq < end && mbar_test(ds_full, nq & 1) && (nq == 0 || mbar_test(dq_empty, (nq - 1) & 1))) {
            tc_fence_after_sync();
            issue_dq(tmem + 384);
            ++nq;
            progressed = true;
          }
          if (acc_ok && nv < np && mbar_test(p_full, nv & 1)) {
            tc_fence_after_sync();
            issue_grad(do_base + (nv % kSpDoStages) * kSpRowBytes, p_addr, tmem + 256, nv == gt, do_empty + (nv % kSpDoStages), p_empty);
            ++nv;
            progressed = true;
          }
          if (ns < end && mbar_test(q_full + (ns % kSpQStages), (ns / kSpQStages) & 1) &&
              (ns < 2 || mbar_test(s_empty + (ns & 1), ((ns >> 1) - 1) & 1))) {
            tc_fence_after_sync();
            issue_logits(q_base + (ns % kSpQStages) * kSpRowBytes, k_addr, tmem + (ns & 1) * KT, s_full + (ns & 1));
            ++ns;
            progressed = true;
          }
          if (acc_ok && nk < np && nk < end && mbar_test(ds_full, nk & 1)) {
            tc_fence_after_sync();
            issue_grad(q_base + (nk % kSpQStages) * kSpRowBytes, ds_addr, tmem + 320, nk == gt, q_empty + (nk % kSpQStages), ds_empty);
            ++nk;
            progressed = true;
          }
          if (np < ns && mbar_test(do_full + (np % kSpDoStages), (np / kSpDoStages) & 1) &&
              (np < 2 || mbar_test(dp_empty + (np & 1), ((np >> 1) - 1) & 1))) {
            tc_fence_after_sync();
            issue_logits(do_base + (np % kSpDoStages) * kSpRowBytes, v_addr, tmem + 128 + (np & 1) * KT, dp_full + (np & 1));
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
              alive = false;
            }
          }
        }
        if (elect_one()) umma_commit(all_done);
        __syncwarp();
        // the K/V tile (read by the last S, dP and dQ products) is replaced at the top of the next item
        if (alive && !mbar_wait(all_done, n_done & 1, p.st)) alive = false;
        gt = end;
        ++n_done;
      }
      cur = nxt;
      item = nitem;
    }
  } else if (warp >= 13) {
    // ===================== dQ drain: lane = d, 128 columns = the rows of the tile =====================
    if (with_dq) {
      constexpr int SPC = 32 >> LOGG;  // tokens (slots) per chunk of 32 columns
      const uint32_t lane_base = tmem + ((uint32_t)((warp & 3) * 32) << 16) + 384;
      int gt = 0;
      bool alive = true;
      int item = take(0);
      SpItem cur = item_or_none(item);
      for (int k = 0; item < n_items && alive; ++k) {
        const int nitem = take(k + 1);
        const SpItem nxt = item_or_none(nitem);
        if (cur.ntiles > 0) {
          const int tok_begin = cur.tok_begin, tok_count = cur.tok_count;
          float* const dst = p.dq32 + (long long)(cur.h * G) * D + (warp & 3) * 32 + lane;
          // one reduction per row: the warp's 32 lanes add 32 consecutive floats of the (token, head) row
          auto reduce_chunk = [&](const uint32_t (&r)[32], int i, int c) {
#pragma unroll
            for (int s2 = 0; s2 < SPC; ++s2) {
              const int ti = i * TPT + c * SPC + s2;
              const int n = ti < tok_count ? __ldg(p.list + tok_begin + ti) : -1;
              if (n >= 0) {
                float* row_dst = dst + (long long)n * p.Hq * D;
#pragma unroll
                for (int g = 0; g < G; ++g) red_add1(row_dst + g * D, r[s2 * G + g]);
              }
            }
          };
          for (int i = 0; i < cur.ntiles; ++i) {
            if (!mbar_wait(dq_full, (gt + i) & 1, p.st)) { alive = false; break; }
            tc_fence_after_sync();
            uint32_t ra[32], rb[32];
            tmem_ld32(lane_base, ra);
            tmem_ld32(lane_base + 32, rb);
            tmem_ld_wait();
            reduce_chunk(ra, i, 0);
            reduce_chunk(rb, i, 1);
            tmem_ld32(lane_base + 64, ra);
            tmem_ld32(lane_base + 96, rb);
            tmem_ld_wait();
            // the rest of the buffer is in registers: the next tile's product may overwrite it
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(dq_empty);
            reduce_chunk(ra, i, 2);
            reduce_chunk(rb, i, 3);
          }
          gt += cur.ntiles;
        }
        cur = nxt;
        item = nitem;
      }
    } else {
      // the queue entries are counted per warp: read them all
      int item = take(0);
      for (int k = 0; item < n_items; ++k) item = take(k + 1);
    }
  } else {
    // ===================== softmax / dS threads: two threads per row (32 of the 64 key columns each) =====================
    const int half = warp >> 2;
    const int row = (warp & 3) * 32 + lane;
    const int slot = row >> logG;
    const uint32_t lane_base = tmem + ((uint32_t)((warp & 3) * 32) << 16);
    const uint32_t prow = smem_u32(p_sm) + row * 128, dsrow = smem_u32(ds_sm) + row * 128;
    int gt = 0, n_done = 0;
    bool alive = true;
    int item = take(0);
    SpItem cur = item_or_none(item);
    for (int k = 0; item < n_items && alive; ++k) {
      const int nitem = take(k + 1);
      const SpItem nxt = item_or_none(nitem);
      if (cur.ntiles > 0) {
        const int ntiles = cur.ntiles, tok_begin = cur.tok_begin, tok_count = cur.tok_count, h = cur.h, qs = cur.qs, kpos = cur.kpos,
                  kvalid = cur.kvalid, krow0 = cur.krow0;
        const int head = h * p.G + (row & (p.G - 1));
        // per-row statistics are fetched ahead: the token of tile i+2, (lse, delta) of tile i+1
        auto token_of = [&](int i) { return (i < ntiles && i * TPT + slot < tok_count) ? __ldg(p.list + tok_begin + i * TPT + slot) : -1; };
        auto stats_of = [&](int n) { return n >= 0 ? __ldg(p.ld + (long long)n * p.Hq + head) : make_float2(INFINITY, 0.f); };
        int n_cur = token_of(0), n_next = token_of(1);
        float2 ld_cur = stats_of(n_cur);
        for (int i = 0; i < ntiles && alive; ++i) {
          const int j = gt + i;
          const int bsel = j & 1;
          const int n_next2 = token_of(i + 2);
          const float2 ld_next = stats_of(n_next);
          // keys of this tile the row may see: those at or before its own position
          int lim = n_cur >= 0 ? max(0, min(kvalid, (n_cur - qs) - kpos + 1)) : 0;
          lim -= half * 32;  // relative to this thread's first column
          const float nlse = -ld_cur.x, ndsc = -ld_cur.y * p.sm_scale;

          // ---- P phase ----
          if (!mbar_wait(s_full + bsel, (j >> 1) & 1, p.st)) { alive = false; break; }
          tc_fence_after_sync();
          float pf[32];
          {
            uint32_t su[32];
            tmem_ld32(lane_base + bsel * KT + half * 32, su);
            tmem_ld_wait();
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(s_empty + bsel);
            // tiles every row of the warp sees in full (all but the block on the diagonal) skip the mask instructions
            if (__all_sync(0xffffffffu, lim >= 32)) {
#pragma unroll
              for (int c2 = 0; c2 < 32; c2 += 2) {
                const float2 x = ffma2(make_float2(__uint_as_float(su[c2]), __uint_as_float(su[c2 + 1])), make_float2(p.scale2, p.scale2),
                                       make_float2(nlse, nlse));
                pf[c2] = fast_exp2(x.x);
                pf[c2 + 1] = fast_exp2(x.y);
              }
            } else {
#pragma unroll
              for (int c2 = 0; c2 < 32; ++c2) pf[c2] = masked_exp2(c2 < lim, fmaf(__uint_as_float(su[c2]), p.scale2, nlse));
            }
            uint32_t pw[16];
#pragma unroll
            for (int c2 = 0; c2 < 16; ++c2) pw[c2] = DT<T>::pack(pf[2 * c2], pf[2 * c2 + 1]);
            if (j > 0) mbar_wait(p_empty, (j - 1) & 1, p.st);  // dV of the previous tile has read the P tile
#pragma unroll
            for (int c4 = 0; c4 < 4; ++c4)
              asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};\n" ::"r"(prow + (((half * 4 + c4) ^ (row & 7)) << 4)), "r"(pw[c4 * 4]),
                           "r"(pw[c4 * 4 + 1]), "r"(pw[c4 * 4 + 2]), "r"(pw[c4 * 4 + 3]) : "memory");
          }
          fence_proxy_async();
          __syncwarp();
          if (lane == 0) mbar_arrive(p_full);

          // ---- dS phase ----
          if (!mbar_wait(dp_full + bsel, (j >> 1) & 1, p.st)) { alive = false; break; }
          tc_fence_after_sync();
          {
            uint32_t du[32];
            tmem_ld32(lane_base + 128 + bsel * KT + half * 32, du);
            tmem_ld_wait();
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(dp_empty + bsel);
            uint32_t dw[16];
#pragma unroll
            for (int c2 = 0; c2 < 32; c2 += 2) {
              const float2 t2 = ffma2(make_float2(__uint_as_float(du[c2]), __uint_as_float(du[c2 + 1])), make_float2(p.sm_scale, p.sm_scale),
                                      make_float2(ndsc, ndsc));
              const float2 d2 = fmul2(make_float2(pf[c2], pf[c2 + 1]), t2);
              dw[c2 >> 1] = DT<T>::pack(d2.x, d2.y);
            }
            if (j > 0) mbar_wait(ds_empty, (j - 1) & 1, p.st);  // dK (and dQ) of the previous tile have read the dS tile
#pragma unroll
            for (int c4 = 0; c4 < 4; ++c4)
              asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};\n" ::"r"(dsrow + (((half * 4 + c4) ^ (row & 7)) << 4)), "r"(dw[c4 * 4]),
                           "r"(dw[c4 * 4 + 1]), "r"(dw[c4 * 4 + 2]), "r"(dw[c4 * 4 + 3]) : "memory");
          }
          fence_proxy_async();
          __syncwarp();
          if (lane == 0) mbar_arrive(ds_full);
          n_cur = n_next;
          n_next = n_next2;
          ld_cur = ld_next;
        }
        if (!alive) break;
        // ---- read out dV and dK of this item: thread (d, half) holds column d for 32 of the 64 keys ----
        if (!mbar_wait(all_done, n_done & 1, p.st)) { alive = false; break; }
        tc_fence_after_sync();
        const int d = row;
        uint32_t rv[32], rk[32];
        tmem_ld32(lane_base + 256 + half * 32, rv);
        tmem_ld32(lane_base + 320 + half * 32, rk);
        tmem_ld_wait();
        // the accumulators are in registers: the next item's dV / dK products may start
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(acc_free);
        float* dstv = p.dv32 + ((size_t)krow0 * p.Hkv + h) * D + d;
        float* dstk = p.dk32 + ((size_t)krow0 * p.Hkv + h) * D + d;
#pragma unroll
        for (int c2 = 0; c2 < 32; ++c2) {
          const int key = half * 32 + c2;
          if (key < kvalid) {
            atomicAdd(dstv + (size_t)key * p.Hkv * D, __uint_as_float(rv[c2]));
            atomicAdd(dstk + (size_t)key * p.Hkv * D, __uint_as_float(rk[c2]));
          }
        }
        gt += ntiles;
        ++n_done;
      }
      cur = nxt;
      item = nitem;
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 12) tmem_dealloc(tmem, 512);
}

template <typename T>
int launch_sparse_dkdv_tc(const void* q, const void* dout, const void* k, const void* v, const long long* strides, int Nk, dim3 grid,
                          DkdvParams p, cudaStream_t stream) {
  constexpr int D = 128;
  int logG = 0;
  while ((1 << logG) < p.G) ++logG;
  CUtensorMap tmK, tmV;
  int rc = make_tmap_3d(&tmK, DT<T>::kTmapType, k, D, p.Hkv, Nk, strides[3], strides[2], 64, 1, 64);
  if (rc) return rc;
  rc = make_tmap_3d(&tmV, DT<T>::kTmapType, v, D, p.Hkv, Nk, strides[5], strides[4], 64, 1, 64);
  if (rc) return rc;
  const size_t smem = 2 * kSpKvBytes + 2 * kSpPdBytes + (kSpQStages + kSpDoStages) * kSpRowBytes + 48 * sizeof(uint64_t) + 64;
  auto launch = [&](auto kern) -> int {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return cuda_rc(e);
    LaunchScope ls_("sparse_dkdv_tc", stream);
    // persistent CTAs: one per SM (shared memory and the 512 TMEM columns allow no more), each taking work items from a
    // grid-wide counter; grid.x * grid.y on entry is the upper bound of their number
    int sms = 148, dev = 0;
    if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    const unsigned long long bound = (unsigned long long)grid.x * grid.y;   // (list entries) x (tiles per block)
    grid = dim3((unsigned)std::min<unsigned long long>(bound, (unsigned long long)sms), 1, 1);
    kern<<<grid, kSpThreads, smem, stream>>>(tmK, tmV, static_cast<const T*>(q), static_cast<const T*>(dout), strides[0], strides[1],
                                             strides[6], strides[7], p);
    return cuda_rc(cudaGetLastError());
  };
  switch (logG) {
    case 2: return launch(sparse_dkdv_tc_kernel<T, 2>);
    case 3: return launch(sparse_dkdv_tc_kernel<T, 3>);
    case 4: return launch(sparse_dkdv_tc_kernel<T, 4>);
    default: return kUnsupported;
  }
}

template int launch_sparse_dkdv_tc<__nv_bfloat16>(const void*, const void*, const void*, const void*, const long long*, int, dim3,
                                                  DkdvParams, cudaStream_t);
template int launch_sparse_dkdv_tc<__half>(const void*, const void*, const void*, const void*, const long long*, int, dim3, DkdvParams,
                                           cudaStream_t);

}  // namespace nsa
