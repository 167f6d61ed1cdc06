// Backward of the compression operators (deterministic: no floating-point atomics).
//
// Linear compression  y = Xwin W + bias(pe, W):
//   dbias[h,n]   = sum_m dy[m,h,n]
//   dW[h,(k,d),n] = sum_m x[s+m*stride+k,h,d] dy[m,h,n] + pe[h,k,d] dbias[h,n]     one CTA per (tap k, head):
//                   a [d x d] tile accumulated over all windows with mma (A = x rows read transposed)
//   dpe[h,(k,d)] = sum_n dbias[h,n] W[h,(k,d),n]
//   dx[t]        = sum_{i < ks/stride} dy[t/stride - i] W_{t%stride + i*stride}^T   grouped by j = t % stride so
//                   that every group is a plain GEMM with the taps on the reduction dimension (overlap-add
//                   happens in registers, not through atomics)
// Pooling:
//   dx[t] = sum_i w[h, j + i*stride] dy[t/stride - i],  dw[h,k] = sum_m <x[s+m*stride+k,h,:], dy[m,h,:]> + <pe[h,k,:], dbias[h,:]>,
//   dpe[h,k,:] = w[h,k] dbias[h,:]
#include "attn_tile.cuh"
#include "dispatch.h"
#include "host_util.h"
#include "nsa_b200.h"
#include "pool_bwd_stream.h"

namespace nsa {

// dbias[h, n] = sum_m dy[m, h, n]   (fp32).  One CTA of 256 threads per (head, 8 columns): a thread walks the rows
// m = tid, tid + 256, ... with one 16-byte load per row; fixed-order reduction (deterministic).
template <typename T>
__global__ void __launch_bounds__(256) colsum_kernel(const T* __restrict__ dy, float* __restrict__ dbias, int M, int H, int D) {
  __shared__ float red[8][8];
  const int h = blockIdx.x, n0 = blockIdx.y * 8;
  float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
  for (int m = threadIdx.x; m < M; m += 256) {
    const uint4 v = __ldg(reinterpret_cast<const uint4*>(dy + ((size_t)m * H + h) * D + n0));
    const uint32_t u[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float2 f = DT<T>::unpack(u[e]);
      acc[2 * e] += f.x;
      acc[2 * e + 1] += f.y;
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
    dbias[h * D + n0 + threadIdx.x] = sum;
  }
}

// dpe[h, r] = sum_n dbias[h, n] * W[h, r, n]
template <typename T>
__global__ void linear_dpe_kernel(const float* __restrict__ dbias, const T* __restrict__ w, T* __restrict__ dpe, int H, int R, int D) {
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= (long long)H * R) return;
  const int h = idx / R;
  const T* wr = w + (size_t)idx * D;
  float acc = 0.f;
  for (int n = 0; n < D; ++n) acc += dbias[h * D + n] * DT<T>::to_float(wr[n]);
  dpe[idx] = DT<T>::from_float(acc);
}

struct LinBwdParams {
  const void* x;
  const void* w;
  const void* pe;
  const void* dy;   // [M, H, D] contiguous
  const float* dbias;
  void* dx;         // [N, H, D] contiguous
  void* dw;         // [H, ks*D, D] contiguous
  const int* cu;
  const int* ycu;
  long long x_sn, x_sh;
  int B, H, ks, stride;
};

// ---- dW: one CTA per (tap, head) ----
template <typename T, int D>
__global__ void __launch_bounds__(D * 2) linear_dw_kernel(LinBwdParams p) {
  constexpr int MT = 64;
  constexpr int TILE = MT * D * 2;
  constexpr int CH = D / 8;
  constexpr int NTHREADS = D * 2;  // D/16 warps, 16 output rows (d) each
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const int warp = threadIdx.x >> 5, l = threadIdx.x & 31;
  const int k = blockIdx.x, h = blockIdx.y;
  const T* x = static_cast<const T*>(p.x);
  const T* dy = static_cast<const T*>(p.dy);

  // flattened list of (sequence, m-tile): walk sequences on the fly
  int b = 0, m0 = 0;
  auto advance_to_valid = [&]() {
    while (b < p.B && m0 >= __ldg(p.ycu + b + 1) - __ldg(p.ycu + b)) { ++b; m0 = 0; }
  };
  auto load_stage = [&](int bb, int mm0, int stg) {
    const uint32_t xa = smem_u32(smem + stg * 2 * TILE);
    const uint32_t ya = xa + TILE;
    const int s0 = __ldg(p.cu + bb), y0 = __ldg(p.ycu + bb), Mb = __ldg(p.ycu + bb + 1) - y0;
    for (int i = threadIdx.x; i < MT * CH; i += NTHREADS) {
      const int r = i / CH, c = i % CH;
      const bool ok = (mm0 + r) < Mb;
      const T* xs = x + (long long)(s0 + (ok ? (mm0 + r) * p.stride + k : 0)) * p.x_sn + (long long)h * p.x_sh + c * 8;
      cp_async16(swz_addr<MT>(xa, r, c), xs, ok);
      const T* ys = dy + ((size_t)(y0 + (ok ? mm0 + r : 0)) * p.H + h) * D + c * 8;
      cp_async16(swz_addr<MT>(ya, r, c), ys, ok);
    }
    cp_async_commit();
  };

  float acc[D / 8][4];
#pragma unroll
  for (int j = 0; j < D / 8; ++j) acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0.f;

  advance_to_valid();
  int stg = 0;
  if (b < p.B) load_stage(b, m0, 0);
  while (b < p.B) {
    int nb = b, nm0 = m0 + MT;
    {  // next tile
      int sb = b, sm0 = m0;
      b = nb; m0 = nm0;
      advance_to_valid();
      nb = b; nm0 = m0;
      b = sb; m0 = sm0;
    }
    if (nb < p.B) {
      load_stage(nb, nm0, stg ^ 1);
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();
    const uint32_t xa = smem_u32(smem + stg * 2 * TILE);
    // A[dd][m] = X[m][dd] read transposed; this warp's rows are dd = 16*warp .. 16*warp+15
#pragma unroll
    for (int kk = 0; kk < MT / 16; ++kk) {
      uint32_t a[1][4];
      ldmatrix_x4_trans(a[0], swz_addr<MT>(xa, kk * 16 + (l & 7) + ((l >> 4) << 3), 2 * warp + ((l >> 3) & 1)));
      mma_kn<T, D / 8, 1, MT>(acc, a, xa + TILE, kk * 16, 0);
    }
    __syncthreads();
    b = nb; m0 = nm0; stg ^= 1;
  }

  // epilogue: + pe[h,k,dd] * dbias[h,n], store dW[h, k*D + dd, n]
  const int r0 = l >> 2, c0 = (l & 3) * 2;
  float pe0 = 0.f, pe1 = 0.f;
  if (p.pe) {
    const T* pe = static_cast<const T*>(p.pe) + ((size_t)h * p.ks + k) * D + warp * 16;
    pe0 = DT<T>::to_float(pe[r0]);
    pe1 = DT<T>::to_float(pe[r0 + 8]);
  }
  T* dw = static_cast<T*>(p.dw) + ((size_t)h * p.ks + k) * D * D + (size_t)warp * 16 * D;
#pragma unroll
  for (int j = 0; j < D / 8; ++j) {
    const int n = j * 8 + c0;
    float b0 = 0.f, b1 = 0.f;
    if (p.pe) { b0 = p.dbias[h * D + n]; b1 = p.dbias[h * D + n + 1]; }
    *reinterpret_cast<uint32_t*>(dw + (size_t)r0 * D + n) = DT<T>::pack(acc[j][0] + pe0 * b0, acc[j][1] + pe0 * b1);
    *reinterpret_cast<uint32_t*>(dw + (size_t)(r0 + 8) * D + n) = DT<T>::pack(acc[j][2] + pe1 * b0, acc[j][3] + pe1 * b1);
  }
}

// ---- dx: CTA = (tile of 64 stride-chunks, phase j, sequence x head) ----
template <typename T, int D>
__global__ void __launch_bounds__(128) linear_dx_kernel(LinBwdParams p) {
  constexpr int CT = 64;
  constexpr int W_BYTES = D * D * 2;
  constexpr int CH = D / 8;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const int warp = threadIdx.x >> 5;
  const int j = blockIdx.y;
  const int b = blockIdx.z / p.H, h = blockIdx.z % p.H;
  const int s0 = __ldg(p.cu + b), L = __ldg(p.cu + b + 1) - s0;
  const int y0 = __ldg(p.ycu + b), Mb = __ldg(p.ycu + b + 1) - y0;
  const int c_base = blockIdx.x * CT;
  if (c_base * p.stride + j >= L) return;
  const int a = p.ks / p.stride;
  const T* w = static_cast<const T*>(p.w) + (size_t)h * p.ks * D * D;
  const T* dy = static_cast<const T*>(p.dy);

  float acc[D / 8][4];
#pragma unroll
  for (int jj = 0; jj < D / 8; ++jj) acc[jj][0] = acc[jj][1] = acc[jj][2] = acc[jj][3] = 0.f;

  for (int i = 0; i < a; ++i) {
    // W_{j + i*stride}: [dd rows][nn contiguous] -> B operand with n = dd, k = nn
    const T* wk = w + (size_t)(j + i * p.stride) * D * D;
    const uint32_t wb = smem_u32(smem);
    __syncthreads();  // previous tap's reads are done
    for (int t = threadIdx.x; t < D * CH; t += 128) {
      const int r = t / CH, c = t % CH;
      cp_async16(swz_addr<D>(wb, r, c), wk + (size_t)r * D + c * 8, true);
    }
    cp_async_commit();
    // A rows: dy[c - i] for c = c_base + 16*warp + r
    uint32_t af[D / 16][4];
    load_a_frags_global<T, D / 16>(af, [&](int r) -> const T* {
      const int m = c_base + warp * 16 + r - i;
      return (m >= 0 && m < Mb) ? dy + ((size_t)(y0 + m) * p.H + h) * D : nullptr;
    });
    cp_async_wait<0>();
    __syncthreads();
    mma_nk<T, D / 8, D / 16, D>(acc, af, wb, 0, 0);
  }
  __syncthreads();
  T* stage = reinterpret_cast<T*>(smem + warp * (16 * (D + 8) * 2));
  T* dx = static_cast<T*>(p.dx);
  const float one[2] = {1.f, 1.f};
  store_rows_staged<T, D>(acc, one, stage, [&](int r) -> T* {
    const int t = (c_base + warp * 16 + r) * p.stride + j;
    return t < L ? dx + ((size_t)(s0 + t) * p.H + h) * D : nullptr;
  });
}

// ------------------------------------------------------------------------------------------------
// pooling backward
// ------------------------------------------------------------------------------------------------
struct PoolBwdParams {
  const void* x;
  const void* w;   // [H, ks] or nullptr
  const void* pe;  // [H, ks, D] or nullptr
  const void* dy;
  const float* dbias;
  void* dx;
  void* dw;   // [H, ks] or nullptr
  void* dpe;  // [H, ks, D] or nullptr
  const int* cu;
  const int* ycu;
  long long x_sn, x_sh;
  int N, B, H, D, ks, stride;
};

template <typename T>
__global__ void __launch_bounds__(256) pool_dx_kernel(PoolBwdParams p) {
  const int CH = p.D / 8;
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= (long long)p.N * p.H * CH) return;
  const int c = idx % CH;
  const int h = (idx / CH) % p.H;
  const int n = idx / ((long long)CH * p.H);
  const int b = find_sequence(p.cu, p.B, n);
  const int t = n - __ldg(p.cu + b);
  const int y0 = __ldg(p.ycu + b), Mb = __ldg(p.ycu + b + 1) - y0;
  const int j = t % p.stride, cq = t / p.stride, a = p.ks / p.stride;
  const T* dy = static_cast<const T*>(p.dy);
  const T* w = p.w ? static_cast<const T*>(p.w) + h * p.ks : nullptr;
  float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  for (int i = 0; i < a; ++i) {
    const int m = cq - i;
    if (m < 0 || m >= Mb) continue;
    const float wv = w ? DT<T>::to_float(w[j + i * p.stride]) : 1.f / (float)p.ks;
    const uint4 v = __ldg(reinterpret_cast<const uint4*>(dy + ((size_t)(y0 + m) * p.H + h) * p.D + c * 8));
    const uint32_t u[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float2 f = DT<T>::unpack(u[e]);
      acc[2 * e] += wv * f.x;
      acc[2 * e + 1] += wv * f.y;
    }
  }
  uint4 out;
  out.x = DT<T>::pack(acc[0], acc[1]);
  out.y = DT<T>::pack(acc[2], acc[3]);
  out.z = DT<T>::pack(acc[4], acc[5]);
  out.w = DT<T>::pack(acc[6], acc[7]);
  *reinterpret_cast<uint4*>(static_cast<T*>(p.dx) + ((size_t)n * p.H + h) * p.D + c * 8) = out;
}

// dw[h,k] (one CTA per (h,k)) and dpe[h,k,:]
template <typename T>
__global__ void __launch_bounds__(256) pool_dw_kernel(PoolBwdParams p) {
  __shared__ float red[8];
  const int h = blockIdx.x, k = blockIdx.y;
  const int CH = p.D / 8;
  const T* x = static_cast<const T*>(p.x);
  const T* dy = static_cast<const T*>(p.dy);
  float acc = 0.f;
  if (p.dw) {
    for (int b = 0; b < p.B; ++b) {
      const int s0 = __ldg(p.cu + b), y0 = __ldg(p.ycu + b), Mb = __ldg(p.ycu + b + 1) - y0;
      for (int i = threadIdx.x; i < Mb * CH; i += blockDim.x) {
        const int m = i / CH, c = i % CH;
        const uint4 xv = __ldg(reinterpret_cast<const uint4*>(x + (long long)(s0 + m * p.stride + k) * p.x_sn + (long long)h * p.x_sh + c * 8));
        const uint4 yv = __ldg(reinterpret_cast<const uint4*>(dy + ((size_t)(y0 + m) * p.H + h) * p.D + c * 8));
        const uint32_t xu[4] = {xv.x, xv.y, xv.z, xv.w}, yu[4] = {yv.x, yv.y, yv.z, yv.w};
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float2 a = DT<T>::unpack(xu[e]), bb = DT<T>::unpack(yu[e]);
          acc += a.x * bb.x + a.y * bb.y;
        }
      }
    }
    if (p.pe)
      for (int n = threadIdx.x; n < p.D; n += blockDim.x)
        acc += DT<T>::to_float(static_cast<const T*>(p.pe)[((size_t)h * p.ks + k) * p.D + n]) * p.dbias[h * p.D + n];
#pragma unroll
    for (int off = 16; off >= 1; off >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, off);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = acc;
    __syncthreads();
    if (threadIdx.x == 0) {
      float tot = 0.f;
      for (int i = 0; i < (int)(blockDim.x >> 5); ++i) tot += red[i];
      static_cast<T*>(p.dw)[h * p.ks + k] = DT<T>::from_float(tot);
    }
  }
  if (p.dpe) {
    const float wv = p.w ? DT<T>::to_float(static_cast<const T*>(p.w)[h * p.ks + k]) : 1.f / (float)p.ks;
    for (int n = threadIdx.x; n < p.D; n += blockDim.x)
      static_cast<T*>(p.dpe)[((size_t)h * p.ks + k) * p.D + n] = DT<T>::from_float(wv * p.dbias[h * p.D + n]);
  }
}

// dw[h,k] from the streaming pass's partial rows (summed in slot order: deterministic) and dpe[h,k,:]
template <typename T>
__global__ void __launch_bounds__(256) pool_dw_finish_kernel(PoolBwdParams p, const float* __restrict__ partial, int nslots) {
  __shared__ float red[8];
  const int h = blockIdx.x, k = blockIdx.y;
  float acc = 0.f;
  for (int s = threadIdx.x; s < nslots; s += blockDim.x) acc += partial[((size_t)s * p.H + h) * p.ks + k];
  if (p.pe)
    for (int n = threadIdx.x; n < p.D; n += blockDim.x)
      acc += DT<T>::to_float(static_cast<const T*>(p.pe)[((size_t)h * p.ks + k) * p.D + n]) * p.dbias[h * p.D + n];
#pragma unroll
  for (int off = 16; off >= 1; off >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, off);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = acc;
  __syncthreads();
  if (threadIdx.x == 0) {
    float tot = 0.f;
    for (int i = 0; i < (int)(blockDim.x >> 5); ++i) tot += red[i];
    static_cast<T*>(p.dw)[h * p.ks + k] = DT<T>::from_float(tot);
  }
  if (p.dpe) {
    const float wv = DT<T>::to_float(static_cast<const T*>(p.w)[h * p.ks + k]);
    for (int n = threadIdx.x; n < p.D; n += blockDim.x)
      static_cast<T*>(p.dpe)[((size_t)h * p.ks + k) * p.D + n] = DT<T>::from_float(wv * p.dbias[h * p.D + n]);
  }
}

template <typename T, int D>
static int run_linear_bwd(LinBwdParams p, void* dpe, float* dbias, int total_y, int max_len, cudaStream_t stream) {
  if (p.pe) {
    { LaunchScope ls_("colsum", stream); colsum_kernel<T><<<dim3(p.H, D / 8), 256, 0, stream>>>(static_cast<const T*>(p.dy), dbias, total_y, p.H, D); }
    p.dbias = dbias;
    const long long hr = (long long)p.H * p.ks * D;
    { LaunchScope ls_("linear_dpe", stream); linear_dpe_kernel<T><<<(unsigned)((hr + 255) / 256), 256, 0, stream>>>(dbias, static_cast<const T*>(p.w),
                                                                          static_cast<T*>(dpe), p.H, p.ks * D, D); }
  }
  {
    const size_t smem = 1024 + 4 * 64 * D * 2;
    auto kern = linear_dw_kernel<T, D>;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return cuda_rc(e);
    { LaunchScope ls_("linear_dw", stream); kern<<<dim3(p.ks, p.H), D * 2, smem, stream>>>(p); }
  }
  {
    const size_t smem = 1024 + D * D * 2;
    auto kern = linear_dx_kernel<T, D>;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return cuda_rc(e);
    const int chunks = (max_len + p.stride - 1) / p.stride;
    { LaunchScope ls_("linear_dx", stream); kern<<<dim3((chunks + 63) / 64, p.stride, p.B * p.H), 128, smem, stream>>>(p); }
  }
  return cuda_rc(cudaGetLastError());
}

template <typename T, int D>
static int run_pool_bwd(PoolBwdParams p, float* dbias, float* partial, long long partial_floats, int total_y, int max_seqlen,
                        int dtype, cudaStream_t stream) {
  if (p.pe) {
    { LaunchScope ls_("colsum", stream); colsum_kernel<T><<<dim3(p.H, D / 8), 256, 0, stream>>>(static_cast<const T*>(p.dy), dbias, total_y, p.H, D); }
    p.dbias = dbias;
  }
  // long inputs: one streaming pass writes dx and (weighted pooling) the partial rows of dw
  const long long need = pool_bwd_stream_partial_floats(p.H, D, p.N, p.B, max_seqlen, p.ks, p.stride);
  if (total_y > 0 && need > 0 && (!p.dw || (partial && partial_floats >= need))) {
    int nslots = 0;
    const int rc = pool_bwd_stream(p.x, p.dw ? p.w : nullptr, p.dy, p.dx, p.dw ? partial : nullptr, &nslots, p.cu, p.ycu, p.B, p.N,
                                   max_seqlen, p.H, D, p.ks, p.stride, p.x_sn, p.x_sh, dtype, stream);
    if (rc != kInvalid && rc != kUnsupported) {
      if (rc) return rc;
      if (p.dw) {
        LaunchScope ls_("pool_dw_finish", stream);
        pool_dw_finish_kernel<T><<<dim3(p.H, p.ks), 256, 0, stream>>>(p, partial, nslots);
      } else if (p.dpe) {
        LaunchScope ls_("pool_dw", stream);
        pool_dw_kernel<T><<<dim3(p.H, p.ks), 256, 0, stream>>>(p);   // average pooling: only dpe is written
      }
      return cuda_rc(cudaGetLastError());
    }
  }
  const long long total = (long long)p.N * p.H * (D / 8);
  { LaunchScope ls_("pool_dx", stream); pool_dx_kernel<T><<<(unsigned)((total + 255) / 256), 256, 0, stream>>>(p); }
  if (p.dw || p.dpe) { LaunchScope ls_("pool_dw", stream); pool_dw_kernel<T><<<dim3(p.H, p.ks), 256, 0, stream>>>(p); }
  return cuda_rc(cudaGetLastError());
}

}  // namespace nsa

extern "C" int nsa_linear_compress_bwd(const void* x, const void* w, const void* pe, const void* dy, const int* cu_seqlens,
                                       const int* y_cu_seqlens, void* dx, void* dw, void* dpe, float* dbias_scratch,
                                       int total_len, int batch, int total_y, int max_seqlen, int num_heads, int head_dim,
                                       int kernel_size, int kernel_stride, long long x_stride_n, long long x_stride_h,
                                       int dtype, void* stream) {
  using namespace nsa;
  if (!x || !w || !cu_seqlens || !y_cu_seqlens || !dx || !dw || batch <= 0 || num_heads <= 0 || total_len <= 0) return kInvalid;
  if (pe && (!dpe || !dbias_scratch)) return kInvalid;
  if (kernel_size <= 0 || kernel_stride <= 0 || kernel_size % kernel_stride || max_seqlen <= 0) return kInvalid;
  if (total_y > 0 && !dy) return kInvalid;
  if ((x_stride_n | x_stride_h) % 8 || !aligned16(x) || !aligned16(w) || !aligned16(dx) || !aligned16(dw)) return kInvalid;
  LinBwdParams p;
  p.x = x; p.w = w; p.pe = pe; p.dy = dy; p.dbias = nullptr; p.dx = dx; p.dw = dw; p.cu = cu_seqlens; p.ycu = y_cu_seqlens;
  p.x_sn = x_stride_n; p.x_sh = x_stride_h; p.B = batch; p.H = num_heads; p.ks = kernel_size; p.stride = kernel_stride;
  return NSA_DISPATCH_T_D(dtype, head_dim, run_linear_bwd, p, dpe, dbias_scratch, total_y, max_seqlen,
                          static_cast<cudaStream_t>(stream));
}

extern "C" long long nsa_pool_compress_bwd_workspace_floats(int total_len, int batch, int max_seqlen, int num_heads, int head_dim,
                                                           int kernel_size, int kernel_stride) {
  if (total_len <= 0 || batch <= 0 || num_heads <= 0 || head_dim <= 0 || kernel_size <= 0 || kernel_stride <= 0) return 0;
  return (long long)num_heads * head_dim +
         nsa::pool_bwd_stream_partial_floats(num_heads, head_dim, total_len, batch, max_seqlen, kernel_size, kernel_stride);
}

extern "C" int nsa_pool_compress_bwd(const void* x, const void* w, const void* pe, const void* dy, const int* cu_seqlens,
                                     const int* y_cu_seqlens, void* dx, void* dw, void* dpe, float* workspace,
                                     long long workspace_floats, int total_len, int batch, int total_y, int max_seqlen,
                                     int num_heads, int head_dim, int kernel_size, int kernel_stride, long long x_stride_n,
                                     long long x_stride_h, int dtype, void* stream) {
  using namespace nsa;
  if (!x || !cu_seqlens || !y_cu_seqlens || !dx || batch <= 0 || num_heads <= 0 || total_len <= 0 || max_seqlen <= 0) return kInvalid;
  // workspace: [H, d] column sums of dy (needed iff pe), then the partial rows of dw of the streaming pass (optional: without
  // them long inputs run on the per-thread kernels)
  const long long dbias_floats = (long long)num_heads * head_dim;
  float* dbias_scratch = workspace && workspace_floats >= dbias_floats ? workspace : nullptr;
  float* partial = workspace && workspace_floats > dbias_floats ? workspace + dbias_floats : nullptr;
  const long long partial_floats = partial ? workspace_floats - dbias_floats : 0;
  if (pe && (!dpe || !dbias_scratch)) return kInvalid;
  if (w && !dw) return kInvalid;
  if (kernel_size <= 0 || kernel_stride <= 0 || kernel_size % kernel_stride) return kInvalid;
  if (total_y > 0 && !dy) return kInvalid;
  if ((x_stride_n | x_stride_h) % 8 || !aligned16(x) || !aligned16(dx)) return kInvalid;
  PoolBwdParams p;
  p.x = x; p.w = w; p.pe = pe; p.dy = dy; p.dbias = nullptr; p.dx = dx; p.dw = w ? dw : nullptr; p.dpe = pe ? dpe : nullptr;
  p.cu = cu_seqlens; p.ycu = y_cu_seqlens; p.x_sn = x_stride_n; p.x_sh = x_stride_h;
  p.N = total_len; p.B = batch; p.H = num_heads; p.D = head_dim; p.ks = kernel_size; p.stride = kernel_stride;
  return NSA_DISPATCH_T_D(dtype, head_dim, run_pool_bwd, p, dbias_scratch, partial, partial_floats, total_y, max_seqlen, dtype,
                          static_cast<cudaStream_t>(stream));
}
