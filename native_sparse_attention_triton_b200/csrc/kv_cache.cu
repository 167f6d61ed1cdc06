// KV-cache maintenance of NSA inference: the three caches of a layer (selected-block keys/values, compressed
// keys/values with their staging buffer of not-yet-compressed tokens, sliding-window ring) and their length counters,
// updated on the device with no host synchronisation.
//
// Replaces NSACache.prepare_compress / update_kv and _fill_kv_cache of the reference
// (native_sparse_attention/module/kv_cache.py:233-449,452-555): a Triton copy kernel sized by `.max().item()` (a host
// synchronisation per call, four calls per prefill) and, per decode step, about twenty indexing launches
// (`torch.where`, advanced-index assignments, in-place counter updates).  Here a prefill fill is one launch per cache
// and a decode step is two launches in all (stage the new token; append to the three caches), each reading the
// counters on the device, so that a decode step can be captured in a CUDA graph.
//
// Every cache is [2 (key, value)][max_batch][rows][heads][head_dim] of 16-bit elements (strides passed in elements,
// head_dim contiguous); the work is pure 16-byte copies, so the element type does not matter.
#include "common.cuh"
#include "host_util.h"
#include "nsa_b200.h"

namespace nsa {

struct CacheView {
  void* base;
  int* len;  // [max_batch] row counters
  long long s2, sb, sn, sh;
  int rows;  // capacity per sequence
};

__device__ __forceinline__ uint4* cache_row(const CacheView& c, int kv, int b, long long row, int h) {
  return reinterpret_cast<uint4*>(static_cast<uint16_t*>(c.base) + kv * c.s2 + b * c.sb + row * c.sn + h * c.sh);
}

struct FillParams {
  CacheView c;
  const void* src[2];
  const int* cu;
  long long src_sn[2], src_sh[2];
  int total, B, H, CH;  // CH = head_dim / 8 chunks of 16 bytes per row
  int mode, a, b;
  Status st;
};

// First source row (relative to its sequence) that goes into the cache, by fill mode.
//   0: the whole sequence; 1: its last `a` rows (sliding window of a rows);
//   2: the rows after the last full compression hop (window a, hop b): what the next compressed token still needs.
__device__ __forceinline__ int fill_first_row(int mode, int a, int b, int len) {
  if (mode == 1) return max(len - a, 0);
  if (mode == 2) return len < a ? 0 : ((len - a) / b + 1) * b;
  return 0;
}

// One warp per source row: lanes copy the row's heads * CH * 2 chunks of 16 bytes.
__global__ void __launch_bounds__(256) cache_fill_kernel(FillParams p) {
  const int lane = threadIdx.x & 31;
  const int warps = (gridDim.x * blockDim.x) >> 5;
  for (int n = (blockIdx.x * blockDim.x + threadIdx.x) >> 5; n < p.total + p.B; n += warps) {
    if (n >= p.total) {  // the B extra items set the counters
      const int b = n - p.total;
      if (lane == 0) {
        const int len = __ldg(p.cu + b + 1) - __ldg(p.cu + b);
        p.c.len[b] = min(len - fill_first_row(p.mode, p.a, p.b, len), p.c.rows);
      }
      continue;
    }
    const int b = find_sequence(p.cu, p.B, n);
    const int s0 = __ldg(p.cu + b), len = __ldg(p.cu + b + 1) - s0;
    const int row = n - s0 - fill_first_row(p.mode, p.a, p.b, len);
    if (row < 0) continue;
    if (row >= p.c.rows) {  // the sequence does not fit: dropped, and reported through the status word
      if (lane == 0) p.st.raise(kErrBadIndex);
      continue;
    }
    const int per_kv = p.H * p.CH;
    for (int it = lane; it < 2 * per_kv; it += 32) {
      const int kv = it / per_kv, rem = it % per_kv, h = rem / p.CH, c = rem % p.CH;
      const uint4 v = __ldg(reinterpret_cast<const uint4*>(static_cast<const uint16_t*>(p.src[kv]) + (long long)n * p.src_sn[kv] +
                                                           (long long)h * p.src_sh[kv]) + c);
      cache_row(p.c, kv, b, row, h)[c] = v;
    }
  }
}

struct StageParams {
  CacheView c;  // staging buffer: rows == window
  const void* src[2];
  long long src_sn[2], src_sh[2];
  int H, CH, window, hop;
};

// Decode, before compression: a buffer that was full (its window was compressed in the previous step) drops its first
// `hop` rows; then the new token is appended.  One CTA per sequence; a thread owns one 16-byte column of the buffer and
// moves it row by row in ascending order, which is safe for a shift towards row 0.
__global__ void __launch_bounds__(256) cache_stage_decode_kernel(StageParams p) {
  const int b = blockIdx.x;
  int len = p.c.len[b];
  __syncthreads();  // every thread has read the counter before thread 0 rewrites it
  const bool shift = len == p.window;
  if (shift) len -= p.hop;
  const int per_kv = p.H * p.CH;
  for (int it = threadIdx.x; it < 2 * per_kv; it += blockDim.x) {
    const int kv = it / per_kv, rem = it % per_kv, h = rem / p.CH, c = rem % p.CH;
    if (shift)
      for (int r = 0; r < len; ++r) cache_row(p.c, kv, b, r, h)[c] = cache_row(p.c, kv, b, r + p.hop, h)[c];
    if (len < p.c.rows)
      cache_row(p.c, kv, b, len, h)[c] = __ldg(reinterpret_cast<const uint4*>(static_cast<const uint16_t*>(p.src[kv]) +
                                                                              (long long)b * p.src_sn[kv] + (long long)h * p.src_sh[kv]) + c);
  }
  if (threadIdx.x == 0) p.c.len[b] = min(len + 1, p.c.rows);
}

struct AppendParams {
  CacheView cmp, sel, win;
  const int* stage_len;  // the staging buffer's counters: a compressed token exists for sequence b iff stage_len[b] == window
  const void* src[3][2];  // [cache][key, value]: one row per sequence
  long long src_sn[3][2], src_sh[3][2];
  int H, CH, window;
  Status st;
};

// Decode, after compression and rotary embedding: append the compressed token (only for sequences whose staging buffer
// is full), the new token to the selected-block cache, and the new token to the sliding-window ring (slot = count mod
// capacity; the counter keeps counting).  One CTA per sequence.
__global__ void __launch_bounds__(256) cache_append_decode_kernel(AppendParams p) {
  const int b = blockIdx.x;
  const int lc = p.cmp.len[b], ls = p.sel.len[b], lw = p.win.len[b];
  const bool has_cmp = __ldg(p.stage_len + b) == p.window;
  __syncthreads();
  const int per_kv = p.H * p.CH;
  const CacheView* views[3] = {&p.cmp, &p.sel, &p.win};
  const long long rows[3] = {lc, ls, lw % p.win.rows};
  const bool ok[3] = {has_cmp && lc < p.cmp.rows, ls < p.sel.rows, true};
  for (int it = threadIdx.x; it < 3 * 2 * per_kv; it += blockDim.x) {
    const int which = it / (2 * per_kv), r2 = it % (2 * per_kv), kv = r2 / per_kv, rem = r2 % per_kv, h = rem / p.CH, c = rem % p.CH;
    if (!ok[which]) continue;
    const uint4 v = __ldg(reinterpret_cast<const uint4*>(static_cast<const uint16_t*>(p.src[which][kv]) +
                                                         (long long)b * p.src_sn[which][kv] + (long long)h * p.src_sh[which][kv]) + c);
    cache_row(*views[which], kv, b, rows[which], h)[c] = v;
  }
  if (threadIdx.x == 0) {
    if (has_cmp) {
      if (lc < p.cmp.rows) p.cmp.len[b] = lc + 1; else p.st.raise(kErrBadIndex);
    }
    if (ls < p.sel.rows) p.sel.len[b] = ls + 1; else p.st.raise(kErrBadIndex);
    p.win.len[b] = lw + 1;
  }
}

static bool view_ok(const CacheView& c) {
  return c.base && c.len && aligned16(c.base) && c.rows > 0 && ((c.s2 | c.sb | c.sn | c.sh) % 8) == 0;
}
static CacheView make_view(void* base, int* len, const long long* s, int rows) {
  CacheView c;
  c.base = base; c.len = len; c.s2 = s[0]; c.sb = s[1]; c.sn = s[2]; c.sh = s[3]; c.rows = rows;
  return c;
}

}  // namespace nsa

extern "C" int nsa_kv_cache_fill(void* cache, int* cache_len, const void* key, const void* value, const int* cu_seqlens,
                                 int mode, int window, int hop, int total_rows, int batch, int cache_rows, int num_heads,
                                 int head_dim, const long long* strides, void* stream) {
  using namespace nsa;
  if (!cu_seqlens || !strides || batch <= 0 || num_heads <= 0 || head_dim <= 0 || head_dim % 8 || total_rows < 0) return kInvalid;
  if (mode < 0 || mode > 2 || (mode >= 1 && window <= 0) || (mode == 2 && (hop <= 0 || window % hop))) return kInvalid;
  FillParams p;
  p.c = make_view(cache, cache_len, strides, cache_rows);
  if (!view_ok(p.c)) return kInvalid;
  p.src[0] = key; p.src[1] = value;
  p.src_sn[0] = strides[4]; p.src_sh[0] = strides[5]; p.src_sn[1] = strides[6]; p.src_sh[1] = strides[7];
  if (total_rows > 0 && (!key || !value || !aligned16(key) || !aligned16(value))) return kInvalid;
  if ((p.src_sn[0] | p.src_sh[0] | p.src_sn[1] | p.src_sh[1]) % 8) return kInvalid;
  p.cu = cu_seqlens; p.total = total_rows; p.B = batch; p.H = num_heads; p.CH = head_dim / 8;
  p.mode = mode; p.a = window; p.b = hop;
  p.st.word = status_word();
  const long long warps = (long long)total_rows + batch;
  const long long blocks = (warps + 7) / 8;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  LaunchScope ls_("kv_cache_fill", s);
  cache_fill_kernel<<<(int)(blocks < 148 * 8 ? blocks : 148 * 8), 256, 0, s>>>(p);
  return cuda_rc(cudaGetLastError());
}

extern "C" int nsa_kv_cache_stage_decode(void* stage_cache, int* stage_len, const void* key, const void* value, int batch,
                                         int kernel_size, int kernel_stride, int num_heads, int head_dim,
                                         const long long* strides, void* stream) {
  using namespace nsa;
  if (!strides || batch <= 0 || num_heads <= 0 || head_dim <= 0 || head_dim % 8) return kInvalid;
  if (kernel_size <= 0 || kernel_stride <= 0 || kernel_size % kernel_stride) return kInvalid;
  StageParams p;
  p.c = make_view(stage_cache, stage_len, strides, kernel_size);
  if (!view_ok(p.c) || !key || !value || !aligned16(key) || !aligned16(value)) return kInvalid;
  p.src[0] = key; p.src[1] = value;
  p.src_sn[0] = strides[4]; p.src_sh[0] = strides[5]; p.src_sn[1] = strides[6]; p.src_sh[1] = strides[7];
  if ((p.src_sn[0] | p.src_sh[0] | p.src_sn[1] | p.src_sh[1]) % 8) return kInvalid;
  p.H = num_heads; p.CH = head_dim / 8; p.window = kernel_size; p.hop = kernel_stride;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  LaunchScope ls_("kv_cache_stage_decode", s);
  cache_stage_decode_kernel<<<batch, 256, 0, s>>>(p);
  return cuda_rc(cudaGetLastError());
}

extern "C" int nsa_kv_cache_append_decode(void* compress_cache, int* compress_len, void* sparse_cache, int* sparse_len,
                                          void* sliding_cache, int* sliding_len, const int* stage_len,
                                          const void* compress_key, const void* compress_value, const void* sparse_key,
                                          const void* sparse_value, const void* sliding_key, const void* sliding_value,
                                          int batch, int kernel_size, int compress_rows, int sparse_rows, int sliding_rows,
                                          int num_heads, int head_dim, const long long* strides, void* stream) {
  using namespace nsa;
  if (!strides || !stage_len || batch <= 0 || num_heads <= 0 || head_dim <= 0 || head_dim % 8 || kernel_size <= 0) return kInvalid;
  AppendParams p;
  p.cmp = make_view(compress_cache, compress_len, strides, compress_rows);
  p.sel = make_view(sparse_cache, sparse_len, strides + 4, sparse_rows);
  p.win = make_view(sliding_cache, sliding_len, strides + 8, sliding_rows);
  if (!view_ok(p.cmp) || !view_ok(p.sel) || !view_ok(p.win)) return kInvalid;
  const void* src[3][2] = {{compress_key, compress_value}, {sparse_key, sparse_value}, {sliding_key, sliding_value}};
  for (int i = 0; i < 3; ++i)
    for (int kv = 0; kv < 2; ++kv) {
      if (!src[i][kv] || !aligned16(src[i][kv])) return kInvalid;
      p.src[i][kv] = src[i][kv];
      p.src_sn[i][kv] = strides[12 + 4 * i + 2 * kv];
      p.src_sh[i][kv] = strides[13 + 4 * i + 2 * kv];
      if ((p.src_sn[i][kv] | p.src_sh[i][kv]) % 8) return kInvalid;
    }
  p.stage_len = stage_len; p.H = num_heads; p.CH = head_dim / 8; p.window = kernel_size;
  p.st.word = status_word();
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  LaunchScope ls_("kv_cache_append_decode", s);
  cache_append_decode_kernel<<<batch, 256, 0, s>>>(p);
  return cuda_rc(cudaGetLastError());
}
