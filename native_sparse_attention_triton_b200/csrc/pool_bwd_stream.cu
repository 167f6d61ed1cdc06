// Backward of weighted / average pooling compression for long inputs, one pass over HBM:
//   dx[c * stride + t] = sum_r w[r * stride + t] * dy[c - r]                  (written once)
//   dw[r * stride + t] = sum_c <dy[c - r], x[c * stride + t]>                 (x read once, dy read once)
// with c the CHUNK of `stride` tokens a row lies in and r < R = kernel / stride the windows that cover the chunk.
// The organisation is the forward's (pool_fwd_stream.cu): a CTA owns a run of chunks of one sequence and one block of heads,
// split into sub-runs, one per group of threads (thread = one 16-byte column group); when dw is wanted a producer lane
// streams the x chunks of every group through that group's ring of shared-memory slots with cp.async.bulk.tensor.  A
// consumer keeps the R gradient rows dy[c], ..., dy[c - R + 1] in registers (one new 16-byte load per chunk), writes the
// chunk's dx rows, and accumulates the kernel_size partial dot products of its 8 columns in registers across its whole
// sub-run; at the end they are summed over the 16 threads of a head and stored as one partial row per (CTA, group, head).
// The caller adds the partial rows in a fixed order (deterministic, no floating-point atomics).
#include <algorithm>

#include "common.cuh"
#include "dispatch.h"
#include "host_util.h"
#include "pool_bwd_stream.h"

namespace nsa {

namespace {
constexpr int kPbConsumers = 256;
constexpr int kPbRingBytes = 192 * 1024;
constexpr int kPbMaxBars = 32;

struct PoolBwdStreamParams {
  const void* w;    // [H, ks] or nullptr
  const void* dy;   // [M, H, D]
  void* dx;         // [N, H, D]
  float* partial;   // [slots][H][ks] or nullptr
  const int* cu;
  const int* ycu;
  int H, D, ks;
  int run, hb, groups, slots;
  Status st;
};

int pb_heads(int H) {
  int hb = 1;
  while (hb * 2 <= H && hb < 8) hb *= 2;
  return hb;
}
int pb_run(int total_len, int stride, int groups) {
  const int chunks = (total_len + stride - 1) / stride;
  return std::max(32 * groups, (chunks + 148 * 4 - 1) / (148 * 4));
}
}  // namespace

template <typename T, int R, int S, bool DW>
__global__ void __launch_bounds__(kPbConsumers + 32, 1) pool_bwd_stream_kernel(const __grid_constant__ CUtensorMap tmX, PoolBwdStreamParams p) {
  extern __shared__ __align__(128) uint8_t smem[];
  constexpr int KS = R * S;
  const int chunk_bytes = S * p.hb * p.D * 2;
  uint8_t* ring = smem;
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + (DW ? (size_t)p.groups * p.slots * chunk_bytes : 0));
  uint64_t* empty = full + kPbMaxBars;
  float* wsm = reinterpret_cast<float*>(empty + kPbMaxBars);   // [hb][KS]

  const int b = blockIdx.y, h0 = blockIdx.z * p.hb;
  const int s0 = __ldg(p.cu + b), L = __ldg(p.cu + b + 1) - s0;
  const int y0 = __ldg(p.ycu + b), Mb = __ldg(p.ycu + b + 1) - y0;
  const int C = (L + S - 1) / S;
  const int c0 = blockIdx.x * p.run;
  if (c0 >= C) return;
  const int nch = min(p.run, C - c0);
  const int per_group = (nch + p.groups - 1) / p.groups;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int CH = p.D / 8;
  const int items = p.hb * CH;
  const int group_warps = items / 32;

  if (DW && threadIdx.x == 0) {
    for (int s = 0; s < p.groups * p.slots; ++s) {
      mbar_init(full + s, 1);
      mbar_init(empty + s, group_warps);
    }
    fence_barrier_init();
  }
  for (int i = threadIdx.x; i < p.hb * KS; i += blockDim.x) {
    const int hh = i / KS;
    wsm[i] = (h0 + hh < p.H) ? (p.w ? DT<T>::to_float(static_cast<const T*>(p.w)[(size_t)(h0 + hh) * KS + (i - hh * KS)]) : 1.f / (float)KS) : 0.f;
  }
  __syncthreads();

  if (warp == kPbConsumers / 32) {
    // ===================== producer (only when dw is wanted): one lane serves the rings of all groups in turn =====================
    if (DW && lane == 0) {
      int issued[8];
      int remaining = 0;
      for (int g = 0; g < p.groups; ++g) {
        issued[g] = 0;
        remaining += max(0, min(nch, (g + 1) * per_group) - g * per_group);
      }
      long long t0 = 0;
      int idle = 0;
      while (remaining > 0) {
        bool progressed = false;
        for (int g = 0; g < p.groups; ++g) {
          const int n = max(0, min(nch, (g + 1) * per_group) - g * per_group);
          const int i = issued[g];
          if (i >= n) continue;
          const int s = g * p.slots + i % p.slots;
          if (i >= p.slots && !mbar_test(empty + s, ((i / p.slots) - 1) & 1)) continue;
          mbar_expect_tx(full + s, chunk_bytes);
          tma_load_3d(ring + (size_t)s * chunk_bytes, &tmX, full + s, 0, h0, s0 + (c0 + g * per_group + i) * S);
          issued[g] = i + 1;
          --remaining;
          progressed = true;
        }
        if (progressed) {
          idle = 0;
        } else if (((++idle) & 255) == 0) {   // bounded wait
          if (idle == 256) t0 = clock64();
          if (clock64() - t0 > (1ll << 30) || (p.st.word && (*reinterpret_cast<volatile int*>(p.st.word) & kErrWaitTimeout))) {
            p.st.raise(kErrWaitTimeout);
            break;
          }
        }
      }
    }
    return;
  }

  // ===================== consumers =====================
  const int g = threadIdx.x / items, col = threadIdx.x - g * items;
  const int hh = col / CH, cc = col - hh * CH;
  const int cg0 = g * per_group, cg1 = min(nch, cg0 + per_group);
  if (cg1 <= cg0) return;
  const bool head_ok = h0 + hh < p.H;
  const int hq = head_ok ? h0 + hh : p.H - 1;   // a thread of a missing head reads a real row and stores nothing
  const T* dyp = static_cast<const T*>(p.dy) + ((size_t)y0 * p.H + hq) * p.D + cc * 8;
  const size_t dy_row = (size_t)p.H * p.D;
  auto load_dy = [&](int m, float2 (&d)[4]) {
    if (m >= 0 && m < Mb) {
      const uint4 v = __ldg(reinterpret_cast<const uint4*>(dyp + (size_t)m * dy_row));
      d[0] = DT<T>::unpack(v.x); d[1] = DT<T>::unpack(v.y); d[2] = DT<T>::unpack(v.z); d[3] = DT<T>::unpack(v.w);
    } else {
      d[0] = d[1] = d[2] = d[3] = make_float2(0.f, 0.f);
    }
  };
  float2 dyr[R][4];   // dyr[r] = dy of window c - r for the current chunk c
#pragma unroll
  for (int r = 1; r < R; ++r) load_dy(c0 + cg0 - r, dyr[r]);
  float2 dwacc[DW ? R : 1][DW ? S : 1];
  if (DW) {
#pragma unroll
    for (int r = 0; r < R; ++r)
#pragma unroll
      for (int t = 0; t < S; ++t) dwacc[DW ? r : 0][DW ? t : 0] = make_float2(0.f, 0.f);
  }
  const float* wrow = wsm + hh * KS;
  const uint8_t* my_ring = ring + (size_t)g * p.slots * chunk_bytes + (size_t)(hh * p.D + cc * 8) * 2;
  const int row_bytes = p.hb * p.D * 2;
  T* dxp = static_cast<T*>(p.dx) + ((size_t)s0 * p.H + hq) * p.D + cc * 8;

  float2 dynext[4];   // the next chunk's new gradient row, fetched one chunk ahead
  load_dy(c0 + cg0, dynext);
  for (int i = 0; i < cg1 - cg0; ++i) {
    const int c = c0 + cg0 + i;
#pragma unroll
    for (int e = 0; e < 4; ++e) dyr[0][e] = dynext[e];
    load_dy(i + 1 < cg1 - cg0 ? c + 1 : -1, dynext);
    const uint8_t* rows = nullptr;
    if (DW) {
      const int s = i % p.slots;
      if (!mbar_wait(full + g * p.slots + s, (i / p.slots) & 1, p.st)) break;
      rows = my_ring + (size_t)s * chunk_bytes;
    }
    const int tok0 = c * S;
#pragma unroll
    for (int t = 0; t < S; ++t) {
      float2 a[4] = {{0.f, 0.f}, {0.f, 0.f}, {0.f, 0.f}, {0.f, 0.f}};
#pragma unroll
      for (int r = 0; r < R; ++r) {
        const float wt = wrow[r * S + t];
        const float2 w2 = make_float2(wt, wt);
#pragma unroll
        for (int e = 0; e < 4; ++e) a[e] = ffma2(w2, dyr[r][e], a[e]);
      }
      if (head_ok && tok0 + t < L) {
        uint4 out;
        out.x = DT<T>::pack(a[0].x, a[0].y);
        out.y = DT<T>::pack(a[1].x, a[1].y);
        out.z = DT<T>::pack(a[2].x, a[2].y);
        out.w = DT<T>::pack(a[3].x, a[3].y);
        *reinterpret_cast<uint4*>(dxp + (size_t)(tok0 + t) * p.H * p.D) = out;
      }
      if (DW) {
        const uint4 v = *reinterpret_cast<const uint4*>(rows + (size_t)t * row_bytes);
        const float2 x0 = DT<T>::unpack(v.x), x1 = DT<T>::unpack(v.y), x2 = DT<T>::unpack(v.z), x3 = DT<T>::unpack(v.w);
#pragma unroll
        for (int r = 0; r < R; ++r) {
          float2 d = dwacc[DW ? r : 0][DW ? t : 0];
          d = ffma2(dyr[r][0], x0, d);
          d = ffma2(dyr[r][1], x1, d);
          d = ffma2(dyr[r][2], x2, d);
          d = ffma2(dyr[r][3], x3, d);
          dwacc[DW ? r : 0][DW ? t : 0] = d;
        }
      }
    }
    if (DW) {
      __syncwarp();
      if (lane == 0) mbar_arrive(empty + g * p.slots + (i % p.slots));
    }
#pragma unroll
    for (int r = R - 1; r > 0; --r)
#pragma unroll
      for (int e = 0; e < 4; ++e) dyr[r][e] = dyr[r - 1][e];
  }

  if (DW) {
    // the 16 threads of a head (consecutive lanes) add their partial dot products; lane cc == 0 stores the row
    const int slot = (blockIdx.y * gridDim.x + blockIdx.x) * p.groups + g;
    float* prow = p.partial + ((size_t)slot * p.H + hq) * KS;
#pragma unroll
    for (int r = 0; r < R; ++r)
#pragma unroll
      for (int t = 0; t < S; ++t) {
        float v = dwacc[DW ? r : 0][DW ? t : 0].x + dwacc[DW ? r : 0][DW ? t : 0].y;
#pragma unroll
        for (int off = 8; off >= 1; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
        if (cc == 0 && head_ok) prow[r * S + t] = v;
      }
  }
}

bool pool_bwd_stream_eligible(int num_heads, int head_dim, int total_len, int kernel_size, int kernel_stride) {
  if (head_dim != 128) return false;          // 16 threads per head row; a 64-element row would make the tensor map swizzle
  if (total_len < 131072) return false;        // short inputs: the per-thread kernels
  if (kernel_size > 32 || (kernel_stride != 8 && kernel_stride != 16)) return false;   // the taps live in registers
  const int R = kernel_size / kernel_stride;
  if (R != 1 && R != 2 && R != 4) return false;
  const int hb = pb_heads(num_heads);
  if (hb < 2) return false;
  const long long chunk = (long long)kernel_stride * hb * head_dim * 2;
  const int groups = kPbConsumers / (hb * (head_dim / 8));
  return groups <= 8 && kPbRingBytes / chunk / groups >= 3;
}

long long pool_bwd_stream_partial_floats(int num_heads, int head_dim, int total_len, int batch, int max_seqlen, int kernel_size,
                                         int kernel_stride) {
  if (!pool_bwd_stream_eligible(num_heads, head_dim, total_len, kernel_size, kernel_stride)) return 0;
  const int hb = pb_heads(num_heads);
  const int groups = kPbConsumers / (hb * (head_dim / 8));
  const int run = pb_run(total_len, kernel_stride, groups);
  const long long ctas = (long long)(((max_seqlen + kernel_stride - 1) / kernel_stride + run - 1) / run) * batch;
  return ctas * groups * num_heads * kernel_size;
}

template <typename T, int D>
static int launch_pool_bwd_stream(const void* x, int* slots_out, int batch, int total_len, int max_seqlen, int stride,
                                  long long x_sn, long long x_sh, PoolBwdStreamParams p, cudaStream_t stream) {
  p.hb = pb_heads(p.H);
  if (batch > 65535) return kUnsupported;   // the batch is a grid dimension here; the caller falls back
  const long long chunk = (long long)stride * p.hb * D * 2;
  p.groups = kPbConsumers / (p.hb * (D / 8));
  p.slots = (int)std::min<long long>(kPbMaxBars / p.groups, kPbRingBytes / chunk / p.groups);
  p.run = pb_run(total_len, stride, p.groups);
  const bool dw = p.w != nullptr && p.partial != nullptr;
  CUtensorMap tmX;
  int rc = make_tmap_3d(&tmX, DT<T>::kTmapType, x, D, p.H, total_len, x_sh, x_sn, D, p.hb, stride);
  if (rc) return rc;
  const dim3 grid(((max_seqlen + stride - 1) / stride + p.run - 1) / p.run, batch, (p.H + p.hb - 1) / p.hb);
  const int nslots = (int)grid.x * batch * p.groups;
  if (slots_out) *slots_out = nslots;
  if (dw) {
    cudaError_t e = cudaMemsetAsync(p.partial, 0, (size_t)nslots * p.H * p.ks * sizeof(float), stream);
    if (e != cudaSuccess) return cuda_rc(e);
  }
  const size_t smem = (dw ? (size_t)p.groups * p.slots * chunk : 0) + 2 * kPbMaxBars * sizeof(uint64_t) + (size_t)p.hb * p.ks * sizeof(float);
  auto launch = [&](auto kern) -> int {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return cuda_rc(e);
    { LaunchScope ls_(dw ? "pool_dx_dw" : "pool_dx", stream); kern<<<grid, kPbConsumers + 32, smem, stream>>>(tmX, p); }
    return cuda_rc(cudaGetLastError());
  };
  const int R = p.ks / stride;
#define NSA_PB_CASE(RR, SS)                                                                   \
  if (R == RR && stride == SS)                                                                \
    return dw ? launch(pool_bwd_stream_kernel<T, RR, SS, true>) : launch(pool_bwd_stream_kernel<T, RR, SS, false>);
  NSA_PB_CASE(1, 16)
  NSA_PB_CASE(2, 16)
  NSA_PB_CASE(2, 8)
  NSA_PB_CASE(4, 8)
#undef NSA_PB_CASE
  return kUnsupported;
}

int pool_bwd_stream(const void* x, const void* w, const void* dy, void* dx, float* partial, int* slots, const int* cu,
                    const int* ycu, int batch, int total_len, int max_seqlen, int num_heads, int head_dim, int kernel_size,
                    int kernel_stride, long long x_sn, long long x_sh, int dtype, cudaStream_t stream) {
  PoolBwdStreamParams p;
  p.w = w; p.dy = dy; p.dx = dx; p.partial = partial; p.cu = cu; p.ycu = ycu; p.H = num_heads; p.D = head_dim; p.ks = kernel_size;
  p.run = p.hb = p.groups = p.slots = 0;
  p.st.word = status_word();
  return NSA_DISPATCH_T_D(dtype, head_dim, launch_pool_bwd_stream, x, slots, batch, total_len, max_seqlen, kernel_stride, x_sn,
                          x_sh, p, stream);
}

}  // namespace nsa
