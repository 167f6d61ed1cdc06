// Linear compression forward as ONE GEMM per (sequence, head) on the 5th-generation tensor cores, operands fed by TMA.
//
//   y[m, :] = sum over taps of  x[s + m * stride + tap, :]  @  W[tap]        (W[tap] is [d x d], d = 128)
//
// A CTA owns 128 consecutive windows m of one (sequence, head) and walks the taps.  For a fixed tap the 128 rows it needs
// are tokens `stride` apart: x is described to TMA as the 4-D tensor [token / stride][token % stride][head][d], so that a box
// of 128 x 1 x 1 x 64 lands those rows densely in shared memory as a K-major, 128-byte-swizzled A panel.  W[tap] arrives
// as two MN-major panels (rows = input feature = reduction index, 64 output features per panel row).  Eight
// 128 x 128 x 16 products per tap accumulate into 128 TMEM columns; the epilogue rounds, adds the position-embedding
// bias in the storage type (as the reference adds its einsum) and stores 16-byte chunks.
//
// The 4-D view covers floor(N / stride) * stride tokens.  The last N % stride tokens are reached through a second tensor
// map whose base is shifted by that remainder: a CTA whose windows touch them uses it (the host only picks this kernel
// when x is long enough that such a CTA never also needs the first N % stride tokens).  Rows of the box beyond the last
// window of the sequence read other tokens or zero fill and are not stored.
//
//   warp 0 : TMA producer     warp 1 : TMEM allocation + MMA issue     warps 2..5 : epilogue (one thread per row)
#include "common.cuh"
#include "dispatch.h"
#include "host_util.h"
#include "linear_fwd_tc.h"
#include "tc5.cuh"

namespace nsa {

namespace {
constexpr int kLinD = 128;
constexpr int kLinRows = 128;
constexpr int kLinStages = 3;
constexpr int kLinPanel = 128 * 128;       // bytes: 128 rows of 64 16-bit elements
constexpr int kLinTile = 2 * kLinPanel;    // one operand of one tap

struct LinTcParams {
  const void* bias;  // [H, 128] or nullptr
  void* y;
  const int* cu;
  const int* ycu;
  int H, ks, stride;
  int groups, rem;   // floor(N / stride), N % stride
  Status st;
};
}  // namespace

template <typename T>
__global__ void __launch_bounds__(192, 1)
linear_fwd_tc_kernel(const __grid_constant__ CUtensorMap tmXa, const __grid_constant__ CUtensorMap tmXb,
                     const __grid_constant__ CUtensorMap tmW, LinTcParams p) {
  extern __shared__ __align__(1024) uint8_t smem[];
  uint8_t* a_sm = smem;                               // [stages][2 panels]
  uint8_t* b_sm = smem + kLinStages * kLinTile;       // [stages][2 panels]
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + 2 * kLinStages * kLinTile);
  uint64_t* full = bars;
  uint64_t* empty = bars + kLinStages;
  uint64_t* acc_full = empty + kLinStages;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_full + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (smem_u32(smem) & 1023u) {  // the swizzled operand tiles need a 1024-byte aligned base
    if (threadIdx.x == 0) p.st.raise(kErrSmemLayout);
    return;
  }
  const int b = blockIdx.y, h = blockIdx.z;
  const int s0 = __ldg(p.cu + b);
  const int y0 = __ldg(p.ycu + b), Mb = __ldg(p.ycu + b + 1) - y0;
  const int m0 = blockIdx.x * kLinRows;
  if (m0 >= Mb) return;
  const int rows = min(kLinRows, Mb - m0);
  // which view of x: the shifted one iff a stored row reads a token beyond the first view
  int tok0 = s0 + m0 * p.stride;
  const bool shifted = tok0 + (rows - 1) * p.stride + p.ks - 1 >= p.groups * p.stride;
  if (shifted) tok0 -= p.rem;
  if (tok0 < 0) {  // excluded by the host's choice of kernel
    if (threadIdx.x == 0) p.st.raise(kErrBadIndex);
    return;
  }
  const CUtensorMap* tmX = shifted ? &tmXb : &tmXa;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kLinStages; ++s) {
      mbar_init(full + s, 1);
      mbar_init(empty + s, 1);
    }
    mbar_init(acc_full, 1);
    fence_barrier_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 128);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = *reinterpret_cast<volatile uint32_t*>(tmem_slot);

  if (warp == 0) {
    // ===================== TMA producer =====================
    if (lane == 0) {
      for (int tap = 0; tap < p.ks; ++tap) {
        const int s = tap % kLinStages;
        if (tap >= kLinStages && !mbar_wait(empty + s, ((tap / kLinStages) - 1) & 1, p.st)) break;
        mbar_expect_tx(full + s, 2 * kLinTile);
        const int tok = tok0 + tap;
        const int g0 = tok / p.stride, j = tok - g0 * p.stride;
#pragma unroll
        for (int pn = 0; pn < 2; ++pn) tma_load_4d(a_sm + s * kLinTile + pn * kLinPanel, tmX, full + s, pn * 64, h, j, g0);
#pragma unroll
        for (int pn = 0; pn < 2; ++pn) tma_load_3d(b_sm + s * kLinTile + pn * kLinPanel, &tmW, full + s, pn * 64, tap * kLinD, h);
      }
    }
  } else if (warp == 1) {
    // ===================== MMA issuer: the warp stays converged, one elected lane issues =====================
    const uint32_t idesc = umma_idesc<T>(128, 128, false, true);
    const uint32_t a_base = smem_u32(a_sm), b_base = smem_u32(b_sm);
    for (int tap = 0; tap < p.ks; ++tap) {
      const int s = tap % kLinStages;
      if (!mbar_wait(full + s, (tap / kLinStages) & 1, p.st)) break;
      tc_fence_after_sync();
      if (elect_one()) {
        const uint32_t a_addr = a_base + s * kLinTile, b_addr = b_base + s * kLinTile;
#pragma unroll
        for (int kk = 0; kk < kLinD / 16; ++kk)
          umma_ss(tmem, umma_desc_kmajor(a_addr + (kk >> 2) * kLinPanel + (kk & 3) * 32),
                  umma_desc_mnmajor(b_addr + kk * 2048, kLinPanel), idesc, tap > 0 || kk > 0);
        umma_commit(empty + s);
      }
      __syncwarp();
    }
    if (elect_one()) umma_commit(acc_full);
    __syncwarp();
  } else {
    // ===================== epilogue: thread = one window =====================
    const int quarter = warp & 3;  // the TMEM lanes a warp may read
    const int r = quarter * 32 + lane;
    mbar_wait(acc_full, 0, p.st);
    tc_fence_after_sync();
    T* yrow = static_cast<T*>(p.y) + ((size_t)(y0 + m0 + r) * p.H + h) * kLinD;
    const T* bias = p.bias ? static_cast<const T*>(p.bias) + (size_t)h * kLinD : nullptr;
#pragma unroll
    for (int c = 0; c < kLinD / 32; ++c) {
      uint32_t v[32];
      tmem_ld32(tmem_addr(tmem, quarter * 32, c * 32), v);
      tmem_ld_wait();
      if (r < rows) {
#pragma unroll
        for (int q4 = 0; q4 < 4; ++q4) {
          float f[8];
#pragma unroll
          for (int e = 0; e < 8; ++e) f[e] = __uint_as_float(v[q4 * 8 + e]);
          if (bias) {
            const uint4 bv = __ldg(reinterpret_cast<const uint4*>(bias + c * 32 + q4 * 8));
            const uint32_t bu[4] = {bv.x, bv.y, bv.z, bv.w};
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const float2 bf = DT<T>::unpack(bu[e]);
              f[2 * e] = DT<T>::to_float(DT<T>::from_float(f[2 * e])) + bf.x;
              f[2 * e + 1] = DT<T>::to_float(DT<T>::from_float(f[2 * e + 1])) + bf.y;
            }
          }
          uint4 out;
          out.x = DT<T>::pack(f[0], f[1]);
          out.y = DT<T>::pack(f[2], f[3]);
          out.z = DT<T>::pack(f[4], f[5]);
          out.w = DT<T>::pack(f[6], f[7]);
          *reinterpret_cast<uint4*>(yrow + c * 32 + q4 * 8) = out;
        }
      }
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem, 128);
}

bool linear_fwd_tc_eligible(int head_dim, int max_y_len, int total_len, int kernel_size, int kernel_stride) {
  // a CTA spans 127 * stride + ks tokens; with twice that many tokens in x a CTA that needs the shifted view never also
  // needs the first (N % stride) tokens
  return head_dim == kLinD && max_y_len >= kLinRows && kernel_stride >= 1 &&
         (long long)total_len >= 2ll * (kLinRows * (long long)kernel_stride + kernel_size);
}

template <typename T, int D>
static int launch_linear_fwd_tc(const void* x, const void* w, int batch, int max_y_len, int total_len, long long x_sn,
                                long long x_sh, LinTcParams p, cudaStream_t stream) {
  if (D != kLinD) return kUnsupported;
  if (batch > 65535) return kUnsupported;   // the batch is a grid dimension here; the caller falls back
  p.groups = total_len / p.stride;
  p.rem = total_len % p.stride;
  CUtensorMap tmXa, tmXb, tmW;
  int rc = make_tmap_4d(&tmXa, DT<T>::kTmapType, x, kLinD, p.H, p.stride, p.groups, x_sh, x_sn, x_sn * p.stride, 64, 1, kLinRows);
  if (rc) return rc;
  rc = make_tmap_4d(&tmXb, DT<T>::kTmapType, static_cast<const T*>(x) + (long long)p.rem * x_sn, kLinD, p.H, p.stride, p.groups,
                    x_sh, x_sn, x_sn * p.stride, 64, 1, kLinRows);
  if (rc) return rc;
  rc = make_tmap_3d(&tmW, DT<T>::kTmapType, w, kLinD, (uint64_t)p.ks * kLinD, p.H, kLinD, (uint64_t)p.ks * kLinD * kLinD, 64, 128, 1);
  if (rc) return rc;
  const size_t smem = 2 * kLinStages * kLinTile + (2 * kLinStages + 1) * sizeof(uint64_t) + 16;
  auto kern = linear_fwd_tc_kernel<T>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return cuda_rc(e);
  dim3 grid((max_y_len + kLinRows - 1) / kLinRows, batch, p.H);
  { LaunchScope ls_("linear_compress_fwd", stream); kern<<<grid, 192, smem, stream>>>(tmXa, tmXb, tmW, p); }
  return cuda_rc(cudaGetLastError());
}

int linear_fwd_tc(const void* x, const void* w, const void* bias, void* y, const int* cu, const int* ycu, int batch,
                  int max_y_len, int total_len, int num_heads, int kernel_size, int kernel_stride, long long x_sn,
                  long long x_sh, int dtype, cudaStream_t stream) {
  LinTcParams p;
  p.bias = bias; p.y = y; p.cu = cu; p.ycu = ycu; p.H = num_heads; p.ks = kernel_size; p.stride = kernel_stride;
  p.groups = p.rem = 0;
  p.st.word = status_word();
  return NSA_DISPATCH_T_D(dtype, kLinD, launch_linear_fwd_tc, x, w, batch, max_y_len, total_len, x_sn, x_sh, p, stream);
}

}  // namespace nsa
