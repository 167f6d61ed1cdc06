// Forward of attention over the selected KV blocks (topk_sparse_attention).
//
// One warp owns one (query token, KV head): its <=16 query heads form the 16 rows of the
// mma tile, so every K/V tile fetched is shared by all heads of the group (the only reuse
// this operator offers).  Each warp runs a private TMA pipeline: the selected blocks are
// turned into a list of 64-key tiles, K and V tiles are fetched with cp.async.bulk.tensor
// straight from the [tokens, kv_heads, d] tensors into 128B-swizzled shared memory, and the
// next tile of each kind is in flight while the current one is used.
// The kernel is bound by L2 -> shared-memory tile fill (16 flop per byte fetched at G = 16).
#include "attn_tile.cuh"
#include "dispatch.h"
#include "host_util.h"
#include "nsa_b200.h"

namespace nsa {

constexpr int kMaxTilesPerQuery = 64;

struct SparseFwdParams {
  const void* q;
  void* o;
  float* lse;  // [N, Hq], base-2 log-sum-exp of the scaled logits
  const int* topk_idx;
  const int* cu_seqlens;
  long long q_sn, q_sh, o_sn, o_sh;
  long long t_sh, t_sn, t_sk;
  int N, B, Hq, Hkv, G, T, block_size;
  float scale2;
  Status st;
};

template <typename T, int D, int WARPS>
__global__ void __launch_bounds__(WARPS * 32, 1)
sparse_fwd_kernel(const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV, SparseFwdParams p) {
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
  int* tiles = reinterpret_cast<int*>(bars + 2 * WARPS) + warp * kMaxTilesPerQuery;

  const int n = blockIdx.x * WARPS + warp;
  if (n >= p.N) return;  // warps are independent: no block-wide barrier below
  const int h = blockIdx.y;
  if (lane == 0) {
    mbar_init(barK, 1);
    mbar_init(barV, 1);
    fence_barrier_init();
  }
  __syncwarp();

  const int b = find_sequence(p.cu_seqlens, p.B, n);
  const int s0 = __ldg(p.cu_seqlens + b);
  const int t = n - s0;
  const int BS = p.block_size;
  const int bq = t / BS;
  const int nsub = BS / kKeyTile;

  // ---- selected blocks -> list of 64-key tiles (in-sequence position of the first key) ----
  int ntiles = 0;
  const int* tptr = p.topk_idx + h * p.t_sh + (long long)n * p.t_sn;
  for (int base = 0; base < p.T; base += 32) {
    const int j = base + lane;
    const int idx = (j < p.T) ? __ldg(tptr + j * p.t_sk) : -1;
    const bool valid = idx >= 0 && idx <= bq;
    const int cnt = valid ? min(nsub, (t - idx * BS) / kKeyTile + 1) : 0;
    int incl = cnt;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      int v = __shfl_up_sync(0xffffffffu, incl, o);
      if (lane >= o) incl += v;
    }
    const int excl = incl - cnt;
    for (int s = 0; s < cnt; ++s) {
      const int pos = ntiles + excl + s;
      if (pos < kMaxTilesPerQuery) tiles[pos] = idx * BS + s * kKeyTile;
    }
    ntiles += __shfl_sync(0xffffffffu, incl, 31);
  }
  if (ntiles > kMaxTilesPerQuery) {
    p.st.raise(kErrBadIndex);
    ntiles = kMaxTilesPerQuery;
  }
  __syncwarp();

  auto issue = [&](bool is_v, int kpos) {
    uint8_t* buf = is_v ? vbuf : kbuf;
    uint64_t* bar = is_v ? barV : barK;
    const CUtensorMap* tm = is_v ? &tmV : &tmK;
    mbar_expect_tx(bar, TILE_BYTES);
#pragma unroll
    for (int pn = 0; pn < PANELS; ++pn) tma_load_3d(buf + pn * (kKeyTile * 128), tm, bar, pn * 64, h, s0 + kpos);
  };
  auto tile_at = [&](int i, int& kpos, int& limv) {
    kpos = tiles[i];
    limv = min(kKeyTile, t - kpos + 1);
  };

  // ---- query fragments: rows = heads of this KV group ----
  const T* qbase = static_cast<const T*>(p.q) + (long long)n * p.q_sn + (long long)h * p.G * p.q_sh;
  uint32_t qf[D / 16][4];
  load_a_frags_global<T, D / 16>(qf, [&](int r) -> const T* { return r < p.G ? qbase + r * p.q_sh : nullptr; });

  float o[D / 8][4];
#pragma unroll
  for (int j = 0; j < D / 8; ++j) o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.f;
  float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
  uint32_t phase = 0;
  warp_attend_tiles<T, D>(qf, o, m, l, ntiles, smem_u32(kbuf), smem_u32(vbuf), barK, barV, phase, p.scale2, p.st, tile_at,
                          issue);

  // ---- epilogue ----
  float rs[2], lse2[2];
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    rs[r] = l[r] > 0.f ? 1.f / l[r] : 0.f;
    lse2[r] = l[r] > 0.f ? m[r] + log2f(l[r]) : -INFINITY;
  }
  if ((lane & 3) == 0) {
    const int r0 = lane >> 2;
    float* lp = p.lse + (long long)n * p.Hq + h * p.G;
    if (r0 < p.G) lp[r0] = lse2[0];
    if (r0 + 8 < p.G) lp[r0 + 8] = lse2[1];
  }
  T* obase = static_cast<T*>(p.o) + (long long)n * p.o_sn + (long long)h * p.G * p.o_sh;
  store_rows_staged<T, D>(o, rs, reinterpret_cast<T*>(kbuf), [&](int r) -> T* { return r < p.G ? obase + r * p.o_sh : nullptr; });
}

template <typename T, int D>
static int launch_sparse_fwd(const void* k, const void* v, long long k_sn, long long k_sh, long long v_sn, long long v_sh,
                             SparseFwdParams p, cudaStream_t stream) {
  constexpr int WARPS = (D == 128) ? 7 : 8;  // as many private K+V tile pairs as shared memory holds
  constexpr int TILE_BYTES = kKeyTile * D * 2;
  CUtensorMap tmK, tmV;
  int rc = make_tmap_3d(&tmK, DT<T>::kTmapType, k, D, p.Hkv, p.N, k_sh, k_sn, 64, 1, kKeyTile);
  if (rc) return rc;
  rc = make_tmap_3d(&tmV, DT<T>::kTmapType, v, D, p.Hkv, p.N, v_sh, v_sn, 64, 1, kKeyTile);
  if (rc) return rc;
  const size_t smem = 1024 + WARPS * 2 * TILE_BYTES + WARPS * 2 * sizeof(uint64_t) + WARPS * kMaxTilesPerQuery * sizeof(int);
  auto kern = sparse_fwd_kernel<T, D, WARPS>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return cuda_rc(e);
  dim3 grid((p.N + WARPS - 1) / WARPS, p.Hkv);
  { LaunchScope ls_("sparse_fwd", stream); kern<<<grid, WARPS * 32, smem, stream>>>(tmK, tmV, p); }
  return cuda_rc(cudaGetLastError());
}

}  // namespace nsa

extern "C" int nsa_topk_sparse_attn_fwd(const void* q, const void* k, const void* v, const int* topk_idx,
                                        const int* cu_seqlens, void* o, float* lse, int total_len, int batch,
                                        int num_q_heads, int num_kv_heads, int head_dim, int topk, int block_size,
                                        const long long* strides, float sm_scale, int dtype, void* stream) {
  using namespace nsa;
  if (!q || !k || !v || !topk_idx || !cu_seqlens || !o || !lse || !strides) return kInvalid;
  if (total_len <= 0 || batch <= 0 || num_kv_heads <= 0 || num_q_heads % num_kv_heads) return kInvalid;
  const int G = num_q_heads / num_kv_heads;
  if (G > 16) return kUnsupported;
  if (block_size < kKeyTile || block_size % kKeyTile) return kUnsupported;
  if (topk <= 0 || (long long)topk * (block_size / kKeyTile) > kMaxTilesPerQuery) return kUnsupported;
  // strides: q_n q_h k_n k_h v_n v_h o_n o_h t_h t_n t_k   (elements)
  SparseFwdParams p;
  p.q = q; p.o = o; p.lse = lse; p.topk_idx = topk_idx; p.cu_seqlens = cu_seqlens;
  p.q_sn = strides[0]; p.q_sh = strides[1]; p.o_sn = strides[6]; p.o_sh = strides[7];
  p.t_sh = strides[8]; p.t_sn = strides[9]; p.t_sk = strides[10];
  p.N = total_len; p.B = batch; p.Hq = num_q_heads; p.Hkv = num_kv_heads; p.G = G; p.T = topk; p.block_size = block_size;
  p.scale2 = sm_scale * kLog2e;
  p.st.word = status_word();
  if ((p.q_sn | p.q_sh | p.o_sn | p.o_sh) % 8 || !aligned16(q) || !aligned16(o)) return kInvalid;
  return NSA_DISPATCH_T_D(dtype, head_dim, launch_sparse_fwd, k, v, strides[2], strides[3], strides[4], strides[5], p,
                          static_cast<cudaStream_t>(stream));
}
