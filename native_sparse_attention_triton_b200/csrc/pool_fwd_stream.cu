// Weighted / average pooling compression forward for long inputs: every token row is fetched from HBM exactly once, in
// large contiguous pieces, by TMA, and read from shared memory exactly once.
//
// A window is kernel_size = R * stride consecutive tokens, so window m is a sum over R consecutive CHUNKS of `stride`
// tokens: y[m] = sum_r P_r[m + r] with P_r[c] = sum_t w[r * stride + t] * x[(c * stride + t)].  A CTA owns a run of
// consecutive windows of one sequence and one block of heads, split into G contiguous sub-runs, one per GROUP of threads
// (a thread = one 16-byte column group of the token rows).  Every group walks its own stream of chunks through its own
// ring of shared-memory slots: a producer lane issues one cp.async.bulk.tensor load per chunk (stride tokens x heads x d:
// 16 KB contiguous in HBM for 4 heads of 128) whenever a slot of any group is free; a consumer thread reads each row of a
// chunk once, feeds it to all R partial sums it belongs to (packed fp32 FMAs), and carries the R - 1 unfinished windows in
// registers from chunk to chunk.  Nothing depends on how many loads the compiler keeps in flight: the rings hold up to
// 128 KB of chunks in flight per SM.  (The per-thread kernel in compress.cu reads every row R times through L1/L2 and is
// used for short inputs, where its latency is lower.)
#include <algorithm>

#include "common.cuh"
#include "dispatch.h"
#include "host_util.h"
#include "pool_fwd_stream.h"

namespace nsa {

namespace {
constexpr int kPoolConsumers = 256;
constexpr int kPoolRingBytes = 192 * 1024;
constexpr int kPoolMaxBars = 32;   // groups x slots per group

struct PoolStreamParams {
  const void* w;     // [H, ks] or nullptr
  const void* bias;  // [H, D] or nullptr
  void* y;
  const int* cu;
  const int* ycu;
  int H, D, ks, stride;
  int run;           // windows per CTA
  int hb;            // heads per CTA
  int groups;        // thread groups (streams) per CTA
  int slots;         // ring slots per group
  Status st;
};
}  // namespace

template <typename T, int R>
__global__ void __launch_bounds__(kPoolConsumers + 32, 1) pool_fwd_stream_kernel(const __grid_constant__ CUtensorMap tmX, PoolStreamParams p) {
  extern __shared__ __align__(128) uint8_t smem[];
  const int chunk_bytes = p.stride * p.hb * p.D * 2;
  uint8_t* ring = smem;                                                  // [groups][slots][chunk]
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + (size_t)p.groups * p.slots * chunk_bytes);
  uint64_t* empty = full + kPoolMaxBars;
  float* wsm = reinterpret_cast<float*>(empty + kPoolMaxBars);           // [hb][ks]

  const int b = blockIdx.y, h0 = blockIdx.z * p.hb;
  const int s0 = __ldg(p.cu + b);
  const int y0 = __ldg(p.ycu + b), Mb = __ldg(p.ycu + b + 1) - y0;
  const int m0 = blockIdx.x * p.run;
  if (m0 >= Mb) return;
  const int nwin = min(p.run, Mb - m0);
  const int per_group = (nwin + p.groups - 1) / p.groups;   // windows of a group (the last groups may have fewer or none)
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int CH = p.D / 8;                  // 16-byte column groups per head
  const int items = p.hb * CH;             // threads of a group
  const int group_warps = items / 32;

  if (threadIdx.x == 0) {
    for (int s = 0; s < p.groups * p.slots; ++s) {
      mbar_init(full + s, 1);
      mbar_init(empty + s, group_warps);
    }
    fence_barrier_init();
  }
  for (int i = threadIdx.x; i < p.hb * p.ks; i += blockDim.x) {
    const int hh = i / p.ks;
    wsm[i] = (p.w && h0 + hh < p.H) ? DT<T>::to_float(static_cast<const T*>(p.w)[(size_t)(h0 + hh) * p.ks + (i - hh * p.ks)]) : 1.f;
  }
  __syncthreads();

  if (warp == kPoolConsumers / 32) {
    // ===================== producer: one lane serves the rings of all groups in turn =====================
    if (lane == 0) {
      int issued[8];
      int remaining = 0;
      for (int g = 0; g < p.groups; ++g) {
        issued[g] = 0;
        const int w0 = g * per_group, w1 = min(nwin, w0 + per_group);
        remaining += w1 > w0 ? (w1 - w0) + R - 1 : 0;
      }
      long long t0 = 0;
      int idle = 0;
      while (remaining > 0) {
        bool progressed = false;
        for (int g = 0; g < p.groups; ++g) {
          const int w0 = g * per_group, w1 = min(nwin, w0 + per_group);
          const int n = w1 > w0 ? (w1 - w0) + R - 1 : 0;
          const int i = issued[g];
          if (i >= n) continue;
          const int s = g * p.slots + i % p.slots;
          if (i >= p.slots && !mbar_test(empty + s, ((i / p.slots) - 1) & 1)) continue;
          mbar_expect_tx(full + s, chunk_bytes);
          tma_load_3d(ring + (size_t)s * chunk_bytes, &tmX, full + s, 0, h0, s0 + (m0 + w0 + i) * p.stride);
          issued[g] = i + 1;
          --remaining;
          progressed = true;
        }
        if (progressed) {
          idle = 0;
        } else if (((++idle) & 255) == 0) {   // bounded: give up after about half a second, or when another CTA already has
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
  const int hh = col / CH, c = col - hh * CH;
  const int w0 = g * per_group, w1 = min(nwin, w0 + per_group);
  if (w1 <= w0) return;
  const int nchunks = (w1 - w0) + R - 1;
  const bool head_ok = h0 + hh < p.H;
  float2 bias2[4] = {{0.f, 0.f}, {0.f, 0.f}, {0.f, 0.f}, {0.f, 0.f}};
  if (p.bias && head_ok) {
    const uint4 bv = __ldg(reinterpret_cast<const uint4*>(static_cast<const T*>(p.bias) + (size_t)(h0 + hh) * p.D + c * 8));
    const uint32_t bu[4] = {bv.x, bv.y, bv.z, bv.w};
#pragma unroll
    for (int e = 0; e < 4; ++e) bias2[e] = DT<T>::unpack(bu[e]);
  }
  const uint8_t* my_ring = ring + (size_t)g * p.slots * chunk_bytes + (size_t)(hh * p.D + c * 8) * 2;
  const int row_bytes = p.hb * p.D * 2;
  const float* wrow = wsm + hh * p.ks;
  const float inv = 1.f / (float)p.ks;
  T* yout = static_cast<T*>(p.y) + ((size_t)(y0 + m0 + w0) * p.H + h0 + hh) * p.D + c * 8;

  float2 acc[R][4];   // acc[r]: the window that is r chunks old
#pragma unroll
  for (int r = 0; r < R; ++r)
#pragma unroll
    for (int e = 0; e < 4; ++e) acc[r][e] = make_float2(0.f, 0.f);

  for (int i = 0; i < nchunks; ++i) {
    const int s = i % p.slots;
    if (!mbar_wait(full + g * p.slots + s, (i / p.slots) & 1, p.st)) break;
    const uint8_t* rows = my_ring + (size_t)s * chunk_bytes;
#pragma unroll 4
    for (int t = 0; t < p.stride; ++t) {
      const uint4 v = *reinterpret_cast<const uint4*>(rows + (size_t)t * row_bytes);
      const float2 x0 = DT<T>::unpack(v.x), x1 = DT<T>::unpack(v.y), x2 = DT<T>::unpack(v.z), x3 = DT<T>::unpack(v.w);
#pragma unroll
      for (int r = 0; r < R; ++r) {
        const float wt = wrow[r * p.stride + t];
        const float2 w2 = make_float2(wt, wt);
        acc[r][0] = ffma2(w2, x0, acc[r][0]);
        acc[r][1] = ffma2(w2, x1, acc[r][1]);
        acc[r][2] = ffma2(w2, x2, acc[r][2]);
        acc[r][3] = ffma2(w2, x3, acc[r][3]);
      }
    }
    // the chunk is consumed: hand the slot back (one arrival per warp of the group)
    __syncwarp();
    if (lane == 0) mbar_arrive(empty + g * p.slots + s);
    // the window that started R - 1 chunks ago is complete
    if (i >= R - 1 && head_ok) {
      float2 o[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        o[e] = acc[R - 1][e];
        if (!p.w) o[e] = make_float2(o[e].x * inv, o[e].y * inv);
        if (p.bias) {
          o[e].x = DT<T>::to_float(DT<T>::from_float(o[e].x)) + bias2[e].x;
          o[e].y = DT<T>::to_float(DT<T>::from_float(o[e].y)) + bias2[e].y;
        }
      }
      uint4 out;
      out.x = DT<T>::pack(o[0].x, o[0].y);
      out.y = DT<T>::pack(o[1].x, o[1].y);
      out.z = DT<T>::pack(o[2].x, o[2].y);
      out.w = DT<T>::pack(o[3].x, o[3].y);
      *reinterpret_cast<uint4*>(yout + (size_t)(i - (R - 1)) * p.H * p.D) = out;
    }
    // age the unfinished windows by one chunk; a new one starts
#pragma unroll
    for (int r = R - 1; r > 0; --r)
#pragma unroll
      for (int e = 0; e < 4; ++e) acc[r][e] = acc[r - 1][e];
#pragma unroll
    for (int e = 0; e < 4; ++e) acc[0][e] = make_float2(0.f, 0.f);
  }
}

// heads per CTA: the largest power of two <= H (at most 8) -- a group is hb * d / 8 threads, one to four warps
static int pool_stream_heads(int H) {
  int hb = 1;
  while (hb * 2 <= H && hb < 8) hb *= 2;
  return hb;
}

bool pool_fwd_stream_eligible(int num_heads, int head_dim, int total_y, int kernel_size, int kernel_stride) {
  if (head_dim != 128) return false;   // a 64-element row would make the tensor map swizzle the chunk
  if (total_y < 8192) return false;    // short inputs: the per-thread kernel has the lower latency
  const int R = kernel_size / kernel_stride;
  if (R != 1 && R != 2 && R != 4 && R != 8) return false;
  const int hb = pool_stream_heads(num_heads);
  if (hb < 2) return false;            // a group is whole warps
  const long long chunk = (long long)kernel_stride * hb * head_dim * 2;
  const int groups = kPoolConsumers / (hb * (head_dim / 8));
  return chunk % 128 == 0 && kPoolRingBytes / chunk / groups >= 3 && groups <= 8;   // a chunk in use and two in flight per group
}

template <typename T, int D>
static int launch_pool_fwd_stream(const void* x, int batch, int total_len, int total_y, int max_y_len, long long x_sn,
                                  long long x_sh, PoolStreamParams p, cudaStream_t stream) {
  p.hb = pool_stream_heads(p.H);
  if (batch > 65535) return kUnsupported;   // the batch is a grid dimension here; the caller falls back
  const long long chunk = (long long)p.stride * p.hb * D * 2;
  p.groups = kPoolConsumers / (p.hb * (D / 8));
  p.slots = (int)std::min<long long>(kPoolMaxBars / p.groups, kPoolRingBytes / chunk / p.groups);
  // about four CTAs per SM over the whole problem; a group re-reads the R - 1 chunks before its sub-run, so sub-runs are
  // kept at 32 windows or more
  p.run = std::max(32 * p.groups, (int)((total_y + 148 * 4 - 1) / (148 * 4)));
  CUtensorMap tmX;
  int rc = make_tmap_3d(&tmX, DT<T>::kTmapType, x, D, p.H, total_len, x_sh, x_sn, D, p.hb, p.stride);
  if (rc) return rc;
  const size_t smem = (size_t)p.groups * p.slots * chunk + 2 * kPoolMaxBars * sizeof(uint64_t) + (size_t)p.hb * p.ks * sizeof(float);
  const dim3 grid((max_y_len + p.run - 1) / p.run, batch, (p.H + p.hb - 1) / p.hb);
  auto launch = [&](auto kern) -> int {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return cuda_rc(e);
    { LaunchScope ls_("pool_compress_fwd", stream); kern<<<grid, kPoolConsumers + 32, smem, stream>>>(tmX, p); }
    return cuda_rc(cudaGetLastError());
  };
  switch (p.ks / p.stride) {
    case 1: return launch(pool_fwd_stream_kernel<T, 1>);
    case 2: return launch(pool_fwd_stream_kernel<T, 2>);
    case 4: return launch(pool_fwd_stream_kernel<T, 4>);
    case 8: return launch(pool_fwd_stream_kernel<T, 8>);
    default: return kUnsupported;
  }
}

int pool_fwd_stream(const void* x, const void* w, const void* bias, void* y, const int* cu, const int* ycu, int batch,
                    int total_len, int total_y, int max_y_len, int num_heads, int head_dim, int kernel_size, int kernel_stride,
                    long long x_sn, long long x_sh, int dtype, cudaStream_t stream) {
  PoolStreamParams p;
  p.w = w; p.bias = bias; p.y = y; p.cu = cu; p.ycu = ycu; p.H = num_heads; p.D = head_dim; p.ks = kernel_size;
  p.stride = kernel_stride; p.run = p.hb = p.groups = p.slots = 0;
  p.st.word = status_word();
  return NSA_DISPATCH_T_D(dtype, head_dim, launch_pool_fwd_stream, x, batch, total_len, total_y, max_y_len, x_sn, x_sh, p, stream);
}

}  // namespace nsa
