// Gated sum of the three branch outputs of an NSA layer and its backward pass.
//
//   out[n, h, :] = gate[n, h, 0] * o_cmp[n, h, :] + gate[n, h, 1] * o_sel[n, h, :] + gate[n, h, 2] * o_win[n, h, :]
//
// The reference evaluates this as three broadcast multiplies and two adds of [N, Hq, d] tensors in eager PyTorch
// (native_sparse_attention/module/native_sparse_attention.py:226-232, infer/nsa_inference.py:146-150), each a full
// pass over HBM with a 16-bit rounding in between.  Here it is one pass: three 16-byte loads, fp32 arithmetic, one
// 16-byte store per thread, so the kernel moves the algorithmic bytes (4 tensors forward, 7 backward) once.
//
// Backward: d_o_i = gate_i * d_out, d_gate[n, h, i] = sum_d d_out[n, h, d] * o_i[n, h, d]; the sum over d runs over
// the head_dim / 8 neighbouring lanes that hold one (token, head) row, by shuffles in a fixed order.
#include "common.cuh"
#include "dispatch.h"
#include "host_util.h"
#include "nsa_b200.h"

namespace nsa {

struct CombineParams {
  const void* gate;
  const void* o[3];
  void* out;           // forward: the sum; backward: unused
  const void* dout;    // backward only
  void* d_gate;        // backward only
  void* d_o[3];        // backward only
  long long g_sn, g_sh, o_sn[3], o_sh[3], out_sn, out_sh, do_sn, do_sh, dg_sn, dg_sh, d_sn[3], d_sh[3];
  long long rows;      // N * H
  int H;
};

__device__ __forceinline__ uint4 ld_stream16(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0, %1, %2, %3}, [%4];\n" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}
__device__ __forceinline__ void st_stream16(void* p, uint4 v) {
  asm volatile("st.global.cs.v4.u32 [%0], {%1, %2, %3, %4};\n" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}

// One thread per 8 consecutive elements of a (token, head) row; CH = D / 8 threads per row.
template <typename T, int D>
__global__ void __launch_bounds__(256) gate_combine_fwd_kernel(CombineParams p) {
  constexpr int CH = D / 8;
  const long long total = p.rows * CH;
  const long long step = (long long)gridDim.x * blockDim.x;
  for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += step) {
    const long long row = idx / CH;
    const int c = (int)(idx % CH);
    const long long n = row / p.H;
    const int h = (int)(row % p.H);
    uint4 v[3];
#pragma unroll
    for (int i = 0; i < 3; ++i) v[i] = ld_stream16(static_cast<const T*>(p.o[i]) + n * p.o_sn[i] + h * p.o_sh[i] + c * 8);
    const T* gp = static_cast<const T*>(p.gate) + n * p.g_sn + h * p.g_sh;
    float g[3];
#pragma unroll
    for (int i = 0; i < 3; ++i) g[i] = DT<T>::to_float(__ldg(gp + i));
    uint4 r;
    uint32_t* rw = reinterpret_cast<uint32_t*>(&r);
#pragma unroll
    for (int w = 0; w < 4; ++w) {
      const float2 a = DT<T>::unpack(reinterpret_cast<const uint32_t*>(&v[0])[w]);
      const float2 b = DT<T>::unpack(reinterpret_cast<const uint32_t*>(&v[1])[w]);
      const float2 d = DT<T>::unpack(reinterpret_cast<const uint32_t*>(&v[2])[w]);
      rw[w] = DT<T>::pack(fmaf(g[2], d.x, fmaf(g[1], b.x, g[0] * a.x)), fmaf(g[2], d.y, fmaf(g[1], b.y, g[0] * a.y)));
    }
    st_stream16(static_cast<T*>(p.out) + n * p.out_sn + h * p.out_sh + c * 8, r);
  }
}

template <typename T, int D>
__global__ void __launch_bounds__(256) gate_combine_bwd_kernel(CombineParams p) {
  constexpr int CH = D / 8;  // 8 or 16 lanes per row: rows never straddle a warp
  const long long total = p.rows * CH;
  const long long step = (long long)gridDim.x * blockDim.x;
  const int lane = threadIdx.x & 31;
  // all 32 lanes of a warp stay in the loop together (the reduction below shuffles across them)
  for (long long base = (long long)blockIdx.x * blockDim.x + (threadIdx.x & ~31); base < total; base += step) {
    const long long idx = base + lane;
    const bool active = idx < total;
    const long long row = active ? idx / CH : 0;
    const int c = (int)(idx % CH);
    const long long n = row / p.H;
    const int h = (int)(row % p.H);
    float dot[3] = {0.f, 0.f, 0.f};
    if (active) {
      const uint4 dv = ld_stream16(static_cast<const T*>(p.dout) + n * p.do_sn + h * p.do_sh + c * 8);
      uint4 v[3];
#pragma unroll
      for (int i = 0; i < 3; ++i) v[i] = ld_stream16(static_cast<const T*>(p.o[i]) + n * p.o_sn[i] + h * p.o_sh[i] + c * 8);
      const T* gp = static_cast<const T*>(p.gate) + n * p.g_sn + h * p.g_sh;
      float2 df[4];
#pragma unroll
      for (int w = 0; w < 4; ++w) df[w] = DT<T>::unpack(reinterpret_cast<const uint32_t*>(&dv)[w]);
#pragma unroll
      for (int i = 0; i < 3; ++i) {
        const float g = DT<T>::to_float(__ldg(gp + i));
        uint4 r;
        uint32_t* rw = reinterpret_cast<uint32_t*>(&r);
        float acc = 0.f;
#pragma unroll
        for (int w = 0; w < 4; ++w) {
          const float2 o2 = DT<T>::unpack(reinterpret_cast<const uint32_t*>(&v[i])[w]);
          acc = fmaf(df[w].x, o2.x, acc);
          acc = fmaf(df[w].y, o2.y, acc);
          rw[w] = DT<T>::pack(g * df[w].x, g * df[w].y);
        }
        dot[i] = acc;
        st_stream16(static_cast<T*>(p.d_o[i]) + n * p.d_sn[i] + h * p.d_sh[i] + c * 8, r);
      }
    }
#pragma unroll
    for (int i = 0; i < 3; ++i)
#pragma unroll
      for (int o = CH / 2; o >= 1; o >>= 1) dot[i] += __shfl_xor_sync(0xffffffffu, dot[i], o);
    if (active && c == 0) {
      T* dg = static_cast<T*>(p.d_gate) + n * p.dg_sn + h * p.dg_sh;
#pragma unroll
      for (int i = 0; i < 3; ++i) dg[i] = DT<T>::from_float(dot[i]);
    }
  }
}

// Enough CTAs to keep every SM's load queues full; the grid-stride loops cover the rest.
static int combine_grid(long long threads_needed) {
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const long long want = (threads_needed + 255) / 256;
  const long long cap = (long long)sms * 16;
  return (int)(want < cap ? (want > 0 ? want : 1) : cap);
}

template <typename T, int D>
static int launch_combine_fwd(CombineParams p, cudaStream_t stream) {
  LaunchScope ls_("gate_combine_fwd", stream);
  gate_combine_fwd_kernel<T, D><<<combine_grid(p.rows * (D / 8)), 256, 0, stream>>>(p);
  return cuda_rc(cudaGetLastError());
}

template <typename T, int D>
static int launch_combine_bwd(CombineParams p, cudaStream_t stream) {
  LaunchScope ls_("gate_combine_bwd", stream);
  gate_combine_bwd_kernel<T, D><<<combine_grid(p.rows * (D / 8)), 256, 0, stream>>>(p);
  return cuda_rc(cudaGetLastError());
}

static bool rows_ok(const void* ptr, long long sn, long long sh) { return ptr && aligned16(ptr) && sn % 8 == 0 && sh % 8 == 0; }

}  // namespace nsa

extern "C" int nsa_gate_combine_fwd(const void* gate, const void* o_cmp, const void* o_sel, const void* o_win, void* out,
                                    int total_len, int num_heads, int head_dim, const long long* strides, int dtype,
                                    void* stream) {
  using namespace nsa;
  if (!gate || !strides || total_len < 0 || num_heads <= 0) return kInvalid;
  if (total_len == 0) return kOk;
  CombineParams p{};
  p.gate = gate; p.o[0] = o_cmp; p.o[1] = o_sel; p.o[2] = o_win; p.out = out;
  p.g_sn = strides[0]; p.g_sh = strides[1];
  for (int i = 0; i < 3; ++i) {
    p.o_sn[i] = strides[2 + 2 * i];
    p.o_sh[i] = strides[3 + 2 * i];
    if (!rows_ok(p.o[i], p.o_sn[i], p.o_sh[i])) return kInvalid;
  }
  p.out_sn = strides[8]; p.out_sh = strides[9];
  if (!rows_ok(out, p.out_sn, p.out_sh)) return kInvalid;
  p.rows = (long long)total_len * num_heads;
  p.H = num_heads;
  return NSA_DISPATCH_T_D(dtype, head_dim, launch_combine_fwd, p, static_cast<cudaStream_t>(stream));
}

extern "C" int nsa_gate_combine_bwd(const void* gate, const void* o_cmp, const void* o_sel, const void* o_win, const void* dout,
                                    void* d_gate, void* d_cmp, void* d_sel, void* d_win, int total_len, int num_heads,
                                    int head_dim, const long long* strides, int dtype, void* stream) {
  using namespace nsa;
  if (!gate || !d_gate || !strides || total_len < 0 || num_heads <= 0) return kInvalid;
  if (total_len == 0) return kOk;
  CombineParams p{};
  p.gate = gate; p.o[0] = o_cmp; p.o[1] = o_sel; p.o[2] = o_win; p.dout = dout; p.d_gate = d_gate;
  p.d_o[0] = d_cmp; p.d_o[1] = d_sel; p.d_o[2] = d_win;
  p.g_sn = strides[0]; p.g_sh = strides[1];
  for (int i = 0; i < 3; ++i) {
    p.o_sn[i] = strides[2 + 2 * i];
    p.o_sh[i] = strides[3 + 2 * i];
    p.d_sn[i] = strides[12 + 2 * i];
    p.d_sh[i] = strides[13 + 2 * i];
    if (!rows_ok(p.o[i], p.o_sn[i], p.o_sh[i]) || !rows_ok(p.d_o[i], p.d_sn[i], p.d_sh[i])) return kInvalid;
  }
  p.do_sn = strides[8]; p.do_sh = strides[9];
  p.dg_sn = strides[10]; p.dg_sh = strides[11];
  if (!rows_ok(dout, p.do_sn, p.do_sh)) return kInvalid;
  p.rows = (long long)total_len * num_heads;
  p.H = num_heads;
  return NSA_DISPATCH_T_D(dtype, head_dim, launch_combine_bwd, p, static_cast<cudaStream_t>(stream));
}
