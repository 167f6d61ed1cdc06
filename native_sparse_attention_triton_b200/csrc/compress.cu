// Strided-window compression of keys / values (forward):
//   linear      y[m,h,:] = concat_k(x[s + m*stride + k, h, :]) @ W[h]  (+ concat_k(pe[h,k,:]) @ W[h])
//   weighted    y[m,h,:] = sum_k w[h,k] * x[s + m*stride + k, h, :]    (+ sum_k w[h,k] * pe[h,k,:])
//   average     weighted with w = 1/kernel_size                        (+ mean_k pe[h,k,:])
// The intra-block position embedding `pe` only contributes a per-head bias, which is computed
// once by a small kernel and added in the epilogue of the main kernel (rounded to the storage
// type first, then added, like the reference's `y + bias`).
//
// Linear compression is a per-head GEMM [windows, kernel_size*d] x [kernel_size*d, d] whose A rows
// are overlapping windows: the K loop walks the kernel taps, the A tile of tap k is the rows
// x[s + m*stride + k] gathered with cp.async into 128B-swizzled shared memory, the B tile is the
// tap's [d, d] slice of W.  Pooling is a vectorised streaming kernel.
#include "attn_tile.cuh"
#include "dispatch.h"
#include "host_util.h"
#include "linear_fwd_tc.h"
#include "pool_fwd_stream.h"
#include "nsa_b200.h"

namespace nsa {

// ------------------------------------------------------------------------------------------------
// bias[h, n] = sum_r a[h, r] * Wm[h, r, n]     (linear: a = pe flattened, Wm = W, R = ks*d, NO = d)
// ------------------------------------------------------------------------------------------------
// One CTA of 256 threads per (head, 8 output columns): a thread walks the rows r = tid, tid + 256, ... with one 16-byte
// load of W per row; the 256 partial sums of each column are reduced in a fixed order (deterministic).
template <typename T>
__global__ void __launch_bounds__(256) linear_bias_kernel(const T* __restrict__ pe, const T* __restrict__ w, T* __restrict__ bias, int R, int NO) {
  __shared__ float red[8][8];
  const int h = blockIdx.x, n0 = blockIdx.y * 8;
  float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
  for (int r = threadIdx.x; r < R; r += 256) {
    const float a = DT<T>::to_float(pe[(size_t)h * R + r]);
    const uint4 wv = __ldg(reinterpret_cast<const uint4*>(w + ((size_t)h * R + r) * NO + n0));
    const uint32_t wu[4] = {wv.x, wv.y, wv.z, wv.w};
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float2 f = DT<T>::unpack(wu[e]);
      acc[2 * e] += a * f.x;
      acc[2 * e + 1] += a * f.y;
    }
  }
#pragma unroll
  for (int j = 0; j < 8; ++j)
#pragma unroll
    for (int off = 16; off >= 1; off >>= 1) acc[j] += __shfl_xor_sync(0xffffffffu, acc[j], off);
  if ((threadIdx.x & 31) == 0)
#pragma unroll
    for (int j = 0; j < 8; ++j) red[threadIdx.x >> 5][j] = acc[j];
  __syncthreads();
  if (threadIdx.x < 8) {
    float sum = 0.f;
#pragma unroll
    for (int wp = 0; wp < 8; ++wp) sum += red[wp][threadIdx.x];
    bias[(size_t)h * NO + n0 + threadIdx.x] = DT<T>::from_float(sum);
  }
}

// bias[h, n] = sum_k wk[h,k] * pe[h,k,n]  (wk == nullptr -> 1/ks)
template <typename T>
__global__ void pool_bias_kernel(const T* __restrict__ pe, const T* __restrict__ wk, T* __restrict__ bias, int ks, int D) {
  const int h = blockIdx.x, n = threadIdx.x;
  if (n >= D) return;
  float acc = 0.f;
  for (int k = 0; k < ks; ++k) {
    const float wv = wk ? DT<T>::to_float(wk[h * ks + k]) : 1.f;
    acc += wv * DT<T>::to_float(pe[((size_t)h * ks + k) * D + n]);
  }
  if (!wk) acc /= (float)ks;
  bias[(size_t)h * D + n] = DT<T>::from_float(acc);
}

// ------------------------------------------------------------------------------------------------
// linear compression forward
// ------------------------------------------------------------------------------------------------
struct LinFwdParams {
  const void* x;
  const void* w;     // [H, ks*D, D] contiguous
  const void* bias;  // [H, D] or nullptr
  void* y;           // [M, H, D] contiguous
  const int* cu;
  const int* ycu;
  long long x_sn, x_sh;
  int H, ks, stride;
};

template <typename T, int D>
__global__ void __launch_bounds__(128) linear_fwd_kernel(LinFwdParams p) {
  constexpr int MT = 64;                      // output rows per CTA
  constexpr int A_BYTES = MT * D * 2;         // [64][D]
  constexpr int B_BYTES = D * D * 2;          // [D][D]
  constexpr int CH = D / 8;                   // 16-byte chunks per row
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const int warp = threadIdx.x >> 5;
  const int b = blockIdx.y, h = blockIdx.z;
  const int s0 = __ldg(p.cu + b);
  const int y0 = __ldg(p.ycu + b), Mb = __ldg(p.ycu + b + 1) - y0;
  const int m0 = blockIdx.x * MT;
  if (m0 >= Mb) return;
  const T* x = static_cast<const T*>(p.x);
  const T* w = static_cast<const T*>(p.w) + (size_t)h * p.ks * D * D;

  auto load_stage = [&](int k, int stg) {
    const uint32_t a_base = smem_u32(smem + stg * (A_BYTES + B_BYTES));
    const uint32_t b_base = a_base + A_BYTES;
    for (int i = threadIdx.x; i < MT * CH; i += 128) {
      const int r = i / CH, c = i % CH;
      const bool ok = (m0 + r) < Mb;
      const T* src = x + (long long)(s0 + (ok ? (m0 + r) * p.stride + k : 0)) * p.x_sn + (long long)h * p.x_sh + c * 8;
      cp_async16(swz_addr<MT>(a_base, r, c), src, ok);
    }
    const T* wk = w + (size_t)k * D * D;
    for (int i = threadIdx.x; i < D * CH; i += 128) {
      const int r = i / CH, c = i % CH;
      cp_async16(swz_addr<D>(b_base, r, c), wk + (size_t)r * D + c * 8, true);
    }
    cp_async_commit();
  };

  float acc[D / 8][4];
#pragma unroll
  for (int j = 0; j < D / 8; ++j) acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0.f;

  load_stage(0, 0);
  for (int k = 0; k < p.ks; ++k) {
    const int stg = k & 1;
    if (k + 1 < p.ks) {
      load_stage(k + 1, stg ^ 1);
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();
    const uint32_t a_base = smem_u32(smem + stg * (A_BYTES + B_BYTES));
    uint32_t af[D / 16][4];
    load_a_frags<D / 16, MT>(af, a_base, warp * 16, 0);
    mma_kn<T, D / 8, D / 16, D>(acc, af, a_base + A_BYTES, 0, 0);
    __syncthreads();
  }

  // epilogue: round, add the bias in the storage type, store
  const int l = lane_id();
  if (p.bias) {
    const T* bias = static_cast<const T*>(p.bias) + (size_t)h * D;
#pragma unroll
    for (int j = 0; j < D / 8; ++j) {
      const int c = j * 8 + (l & 3) * 2;
      const float b0 = DT<T>::to_float(bias[c]), b1 = DT<T>::to_float(bias[c + 1]);
#pragma unroll
      for (int e = 0; e < 4; ++e)
        acc[j][e] = DT<T>::to_float(DT<T>::from_float(acc[j][e])) + ((e & 1) ? b1 : b0);
    }
  }
  T* stage = reinterpret_cast<T*>(smem + warp * (16 * (D + 8) * 2));
  T* ybase = static_cast<T*>(p.y) + ((size_t)(y0 + m0 + warp * 16) * p.H + h) * D;
  const float one[2] = {1.f, 1.f};
  store_rows_staged<T, D>(acc, one, stage, [&](int r) -> T* {
    return (m0 + warp * 16 + r < Mb) ? ybase + (size_t)r * p.H * D : nullptr;
  });
}

// ------------------------------------------------------------------------------------------------
// pooling forward (weighted or average): one thread per (window, head, 8-element chunk)
// ------------------------------------------------------------------------------------------------
struct PoolFwdParams {
  const void* x;
  const void* w;     // [H, ks] or nullptr (average)
  const void* bias;  // [H, D] or nullptr
  void* y;
  const int* cu;
  const int* ycu;
  long long x_sn, x_sh;
  int B, H, D, ks, stride, M;
};

template <typename T, int TAPS>
__global__ void __launch_bounds__(256) pool_fwd_kernel(PoolFwdParams p) {
  const int CH = p.D / 8;
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const long long total = (long long)p.M * p.H * CH;
  if (idx >= total) return;
  const int c = idx % CH;
  const int h = (idx / CH) % p.H;
  const int mg = idx / ((long long)CH * p.H);
  const int b = find_sequence(p.ycu, p.B, mg);
  const int m = mg - __ldg(p.ycu + b);
  const T* x = static_cast<const T*>(p.x) + (long long)(__ldg(p.cu + b) + m * p.stride) * p.x_sn + (long long)h * p.x_sh + c * 8;
  const T* w = p.w ? static_cast<const T*>(p.w) + h * p.ks : nullptr;
  float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  // TAPS taps per step (kernel sizes are multiples of 16): eight independent 16-byte loads in flight per thread keep HBM
  // busy on long inputs; the few rows of a decode step take sixteen, so that a window costs one or two memory round trips
  for (int k0 = 0; k0 < p.ks; k0 += TAPS) {
    uint4 v[TAPS];
    float wv[TAPS];
#pragma unroll
    for (int u = 0; u < TAPS; ++u) {
      v[u] = __ldg(reinterpret_cast<const uint4*>(x + (long long)(k0 + u) * p.x_sn));
      wv[u] = w ? DT<T>::to_float(w[k0 + u]) : 1.f;
    }
#pragma unroll
    for (int u = 0; u < TAPS; ++u) {
      const uint32_t uu[4] = {v[u].x, v[u].y, v[u].z, v[u].w};
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float2 f = DT<T>::unpack(uu[e]);
        acc[2 * e] += wv[u] * f.x;
        acc[2 * e + 1] += wv[u] * f.y;
      }
    }
  }
  if (!w) {
    const float inv = 1.f / (float)p.ks;
#pragma unroll
    for (int e = 0; e < 8; ++e) acc[e] *= inv;
  }
  if (p.bias) {
    const T* bias = static_cast<const T*>(p.bias) + (size_t)h * p.D + c * 8;
#pragma unroll
    for (int e = 0; e < 8; ++e) acc[e] = DT<T>::to_float(DT<T>::from_float(acc[e])) + DT<T>::to_float(bias[e]);
  }
  uint4 out;
  out.x = DT<T>::pack(acc[0], acc[1]);
  out.y = DT<T>::pack(acc[2], acc[3]);
  out.z = DT<T>::pack(acc[4], acc[5]);
  out.w = DT<T>::pack(acc[6], acc[7]);
  *reinterpret_cast<uint4*>(static_cast<T*>(p.y) + ((size_t)mg * p.H + h) * p.D + c * 8) = out;
}

// ------------------------------------------------------------------------------------------------
// pooling of the staged rows of a decode step: K and V in one launch
// ------------------------------------------------------------------------------------------------
// Each sequence contributes exactly one window: the kernel_size rows of its staging buffer.  No cu_seqlens, no sequence
// search: the only loads are the rows, the weights and the bias, all independent of each other (one memory round trip; with
// cold caches the general kernel's chain of dependent loads costs 10 us per launch).
struct PoolPairParams {
  const void* x[2];     // [B, ks, H, D] views (strides x_sb, x_sn, x_sh)
  const void* w[2];     // [H, ks] or nullptr (average)
  const void* bias[2];  // [H, D] or nullptr
  void* y[2];           // [B, H, D] contiguous
  long long x_sb, x_sn, x_sh;
  int B, H, D, ks;
};

template <typename T>
__global__ void __launch_bounds__(256) pool_decode_pair_kernel(PoolPairParams p) {
  const int which = blockIdx.y;
  const int CH = p.D / 8;
  const int idx = blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= p.B * p.H * CH) return;
  const int c = idx % CH;
  const int h = (idx / CH) % p.H;
  const int b = idx / (CH * p.H);
  const T* x = static_cast<const T*>(p.x[which]) + (long long)b * p.x_sb + (long long)h * p.x_sh + c * 8;
  const T* w = p.w[which] ? static_cast<const T*>(p.w[which]) + h * p.ks : nullptr;
  uint4 bv = make_uint4(0u, 0u, 0u, 0u);
  if (p.bias[which]) bv = __ldg(reinterpret_cast<const uint4*>(static_cast<const T*>(p.bias[which]) + (size_t)h * p.D + c * 8));
  float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  for (int k0 = 0; k0 < p.ks; k0 += 16) {
    uint4 v[16];
    float wv[16];
#pragma unroll
    for (int u = 0; u < 16; ++u) {
      v[u] = __ldg(reinterpret_cast<const uint4*>(x + (long long)(k0 + u) * p.x_sn));
      wv[u] = w ? DT<T>::to_float(w[k0 + u]) : 1.f;
    }
#pragma unroll
    for (int u = 0; u < 16; ++u) {
      const uint32_t uu[4] = {v[u].x, v[u].y, v[u].z, v[u].w};
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float2 f = DT<T>::unpack(uu[e]);
        acc[2 * e] += wv[u] * f.x;
        acc[2 * e + 1] += wv[u] * f.y;
      }
    }
  }
  if (!w) {
    const float inv = 1.f / (float)p.ks;
#pragma unroll
    for (int e = 0; e < 8; ++e) acc[e] *= inv;
  }
  if (p.bias[which]) {
    const uint32_t bu[4] = {bv.x, bv.y, bv.z, bv.w};
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float2 f = DT<T>::unpack(bu[e]);
      acc[2 * e] = DT<T>::to_float(DT<T>::from_float(acc[2 * e])) + f.x;
      acc[2 * e + 1] = DT<T>::to_float(DT<T>::from_float(acc[2 * e + 1])) + f.y;
    }
  }
  uint4 out;
  out.x = DT<T>::pack(acc[0], acc[1]);
  out.y = DT<T>::pack(acc[2], acc[3]);
  out.z = DT<T>::pack(acc[4], acc[5]);
  out.w = DT<T>::pack(acc[6], acc[7]);
  *reinterpret_cast<uint4*>(static_cast<T*>(p.y[which]) + ((size_t)b * p.H + h) * p.D + c * 8) = out;
}

template <typename T, int D>
static int launch_pool_decode_pair(PoolPairParams p, cudaStream_t stream) {
  const int total = p.B * p.H * (D / 8);
  { LaunchScope ls_("pool_compress_decode", stream); pool_decode_pair_kernel<T><<<dim3((total + 255) / 256, 2), 256, 0, stream>>>(p); }
  return cuda_rc(cudaGetLastError());
}

template <typename T, int D>
static int launch_pool_bias(const void* pe, const void* w, void* bias, int H, int ks, cudaStream_t stream) {
  { LaunchScope ls_("pool_bias", stream); pool_bias_kernel<T><<<H, D, 0, stream>>>(static_cast<const T*>(pe), static_cast<const T*>(w), static_cast<T*>(bias), ks, D); }
  return cuda_rc(cudaGetLastError());
}

template <typename T, int D>
static int launch_linear_fwd(LinFwdParams p, const void* pe, void* bias_scratch, int B, int max_ylen, int total_len, int dtype,
                             cudaStream_t stream) {
  if (pe) {
    { LaunchScope ls_("linear_bias", stream); linear_bias_kernel<T><<<dim3(p.H, D / 8), 256, 0, stream>>>(
        static_cast<const T*>(pe), static_cast<const T*>(p.w), static_cast<T*>(bias_scratch), p.ks * D, D); }
    p.bias = bias_scratch;
  } else {
    p.bias = nullptr;
  }
  if (linear_fwd_tc_eligible(D, max_ylen, total_len, p.ks, p.stride)) {
    const int rc = linear_fwd_tc(p.x, p.w, p.bias, p.y, p.cu, p.ycu, B, max_ylen, total_len, p.H, p.ks, p.stride, p.x_sn, p.x_sh,
                                 dtype, stream);
    if (rc != kInvalid && rc != kUnsupported) return rc;   // a view of x no tensor map describes: the gathering kernel below
  }
  const size_t smem = 1024 + 2 * (64 * D * 2 + D * D * 2);
  auto kern = linear_fwd_kernel<T, D>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return cuda_rc(e);
  dim3 grid((max_ylen + 63) / 64, B, p.H);
  { LaunchScope ls_("linear_compress_fwd", stream); kern<<<grid, 128, smem, stream>>>(p); }
  return cuda_rc(cudaGetLastError());
}

template <typename T, int D>
static int launch_pool_fwd(PoolFwdParams p, const void* pe, void* bias_scratch, int total_len, int max_y_len, int dtype,
                           cudaStream_t stream) {
  if (pe) {
    { LaunchScope ls_("pool_bias", stream); pool_bias_kernel<T><<<p.H, D, 0, stream>>>(static_cast<const T*>(pe), static_cast<const T*>(p.w),
                                                static_cast<T*>(bias_scratch), p.ks, D); }
    p.bias = bias_scratch;
  } else {
    p.bias = nullptr;
  }
  if (pool_fwd_stream_eligible(p.H, D, p.M, p.ks, p.stride)) {
    const int rc = pool_fwd_stream(p.x, p.w, p.bias, p.y, p.cu, p.ycu, p.B, total_len, p.M, max_y_len, p.H, D, p.ks, p.stride,
                                   p.x_sn, p.x_sh, dtype, stream);
    if (rc != kInvalid && rc != kUnsupported) return rc;   // a view of x no tensor map describes: the per-thread kernel below
  }
  const long long total = (long long)p.M * p.H * (D / 8);
  const int blocks = (int)((total + 255) / 256);
  {
    LaunchScope ls_("pool_compress_fwd", stream);
    if (blocks <= 148) pool_fwd_kernel<T, 16><<<blocks, 256, 0, stream>>>(p);   // latency-bound: fewer, wider steps
    else pool_fwd_kernel<T, 8><<<blocks, 256, 0, stream>>>(p);
  }
  return cuda_rc(cudaGetLastError());
}

}  // namespace nsa

extern "C" int nsa_linear_compress_fwd(const void* x, const void* w, const void* pe, const int* cu_seqlens,
                                       const int* y_cu_seqlens, void* y, void* bias_scratch, int total_len, int batch,
                                       int total_y, int max_y_len, int num_heads, int head_dim, int kernel_size,
                                       int kernel_stride, long long x_stride_n, long long x_stride_h, int dtype,
                                       void* stream) {
  using namespace nsa;
  if (!x || !w || !cu_seqlens || !y_cu_seqlens || batch <= 0 || num_heads <= 0) return kInvalid;
  if (pe && !bias_scratch) return kInvalid;
  if (kernel_size <= 0 || kernel_stride <= 0 || kernel_size % kernel_stride) return kInvalid;
  if (total_y <= 0 || max_y_len <= 0) return kOk;  // every sequence is shorter than the window
  if (!y) return kInvalid;
  if ((x_stride_n | x_stride_h) % 8 || !aligned16(x) || !aligned16(w) || !aligned16(y)) return kInvalid;
  LinFwdParams p;
  p.x = x; p.w = w; p.bias = nullptr; p.y = y; p.cu = cu_seqlens; p.ycu = y_cu_seqlens;
  p.x_sn = x_stride_n; p.x_sh = x_stride_h; p.H = num_heads; p.ks = kernel_size; p.stride = kernel_stride;
  return NSA_DISPATCH_T_D(dtype, head_dim, launch_linear_fwd, p, pe, bias_scratch, batch, max_y_len, total_len, dtype,
                          static_cast<cudaStream_t>(stream));
}

extern "C" int nsa_pool_compress_fwd(const void* x, const void* w, const void* pe, const int* cu_seqlens,
                                     const int* y_cu_seqlens, void* y, void* bias_scratch, int total_len, int batch,
                                     int total_y, int max_y_len, int num_heads, int head_dim, int kernel_size, int kernel_stride,
                                     long long x_stride_n, long long x_stride_h, int dtype, void* stream) {
  using namespace nsa;
  if (!x || !cu_seqlens || !y_cu_seqlens || batch <= 0 || num_heads <= 0) return kInvalid;
  if (pe && !bias_scratch) return kInvalid;
  if (kernel_size <= 0 || kernel_stride <= 0 || kernel_size % kernel_stride) return kInvalid;
  if (kernel_size % 16) return kUnsupported;  // the kernel reads sixteen or eight taps per step
  if (total_y <= 0) return kOk;
  if (!y) return kInvalid;
  if ((x_stride_n | x_stride_h) % 8 || !aligned16(x) || !aligned16(y)) return kInvalid;
  PoolFwdParams p;
  p.x = x; p.w = w; p.bias = nullptr; p.y = y; p.cu = cu_seqlens; p.ycu = y_cu_seqlens;
  p.x_sn = x_stride_n; p.x_sh = x_stride_h; p.B = batch; p.H = num_heads; p.D = head_dim; p.ks = kernel_size;
  p.stride = kernel_stride; p.M = total_y;
  return NSA_DISPATCH_T_D(dtype, head_dim, launch_pool_fwd, p, pe, bias_scratch, total_len, max_y_len, dtype,
                          static_cast<cudaStream_t>(stream));
}

extern "C" int nsa_pool_bias(const void* pe, const void* w, void* bias, int num_heads, int head_dim, int kernel_size, int dtype,
                             void* stream) {
  using namespace nsa;
  if (!pe || !bias || num_heads <= 0 || kernel_size <= 0) return kInvalid;
  return NSA_DISPATCH_T_D(dtype, head_dim, launch_pool_bias, pe, w, bias, num_heads, kernel_size, static_cast<cudaStream_t>(stream));
}

extern "C" int nsa_pool_compress_decode_pair(const void* x_k, const void* x_v, const void* w_k, const void* w_v, const void* bias_k,
                                             const void* bias_v, void* y_k, void* y_v, int batch, int num_heads, int head_dim,
                                             int kernel_size, long long x_stride_b, long long x_stride_n, long long x_stride_h,
                                             int dtype, void* stream) {
  using namespace nsa;
  if (!x_k || !x_v || !y_k || !y_v || batch <= 0 || num_heads <= 0 || kernel_size <= 0) return kInvalid;
  if (kernel_size % 16) return kUnsupported;
  if ((x_stride_b | x_stride_n | x_stride_h) % 8 || !aligned16(x_k) || !aligned16(x_v) || !aligned16(y_k) || !aligned16(y_v)) return kInvalid;
  if ((bias_k && !aligned16(bias_k)) || (bias_v && !aligned16(bias_v))) return kInvalid;
  PoolPairParams p;
  p.x[0] = x_k; p.x[1] = x_v; p.w[0] = w_k; p.w[1] = w_v; p.bias[0] = bias_k; p.bias[1] = bias_v; p.y[0] = y_k; p.y[1] = y_v;
  p.x_sb = x_stride_b; p.x_sn = x_stride_n; p.x_sh = x_stride_h; p.B = batch; p.H = num_heads; p.D = head_dim; p.ks = kernel_size;
  return NSA_DISPATCH_T_D(dtype, head_dim, launch_pool_decode_pair, p, static_cast<cudaStream_t>(stream));
}
